// Error convention and small helpers of the host side (reference: src/reef/util/common.h:8-65).
#pragma once
#include <cstdio>
#include <cstdlib>

namespace reef {

// Same values as the reference enum and as the reef_status ints of the C-ABI.
enum Status { Succ = 0, Fail = 1, NotFound = 2, OutOfRange = 3, Full = 4, Timeout = 5 };

void log_error(const char* what, const char* file, int line);

#define RETURN_STATUS(cmd)                                         \
    {                                                              \
        ::reef::Status _s = (::reef::Status)(cmd);                 \
        if (_s != ::reef::Status::Succ) {                          \
            ::reef::log_error(#cmd, __FILE__, __LINE__);           \
            return _s;                                             \
        }                                                          \
    }

// Device-layer calls return the same integers; a failure is reported and propagated as Fail
// unless it is one of the enum values already (reference: GPU_RETURN_STATUS, hip_impl.h:25-32).
#define GPU_RETURN_STATUS(cmd) RETURN_STATUS(cmd)

template <typename T>
T align_up(T value, T alignment) {
    T temp = value % alignment;
    return temp == 0 ? value : value - temp + alignment;
}
template <typename T>
T align_down(T value, T alignment) {
    return value - value % alignment;
}

}  // namespace reef
