/*
 * Development aids of libreef_cuda.  These entry points exist only in a library built with -DREEF_DEBUG_AIDS
 * (REEF_DEBUG_AIDS=1 python -m reef_b200.build); the default library neither exports them nor carries the stamps in
 * its kernels.  The same switch lets the scheduler read its padding parameters from REEF_PAD_* environment variables
 * and print its padding-loop statistics.  No reference counterpart (the reference has wall-clock stamps only,
 * src/reef/server/scheduler.h:54-56).
 */
#ifndef REEF_DEBUG_AIDS_H_
#define REEF_DEBUG_AIDS_H_

#include "reef_cuda.h"

#ifdef __cplusplus
extern "C" {
#endif

/* Phase trace of the tensor-core convolution.  While enabled, block (0,0) of every tensor-core launch records the SM
 * clock at {0 entry, 1 set-up done, 2 ring filled, 3 peers up, 4 first K block landed, 5 last K block landed,
 * 6 accumulator complete, 7 tile staged, 8 exchange complete, 9 rows finished, 10 leaving};
 * reef_trace_read copies the 16-word record of the latest launch (call after synchronising). */
REEF_API reef_status reef_trace_enable(int on);
REEF_API reef_status reef_trace_read(int64_t* stamps16);

#ifdef __cplusplus
}
#endif
#endif /* REEF_DEBUG_AIDS_H_ */
