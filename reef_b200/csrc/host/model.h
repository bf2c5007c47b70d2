// Model resources: <model>.json schedule graph, <model>.profile.json latency tables and the
// <model>.param blob (reference: src/reef/executor/model.h:14-70, model.cpp:13-156).
#pragma once
#include <cstddef>
#include <cstdint>
#include <memory>
#include <string>
#include <unordered_map>
#include <vector>

#include "common.h"

namespace reef {
namespace executor {

class StorageInfo {
public:
    std::string name;
    size_t size;          // elements
    std::string stype;    // float32 | int64 | byte | uint1 | int32
};

class KernelInfo {
public:
    std::string name;
    uint32_t launch_params[6];   // grid x,y,z, block x,y,z
    std::vector<size_t> args;    // storage indices, positional
};

class Model {
public:
    std::vector<StorageInfo> storage;
    std::vector<KernelInfo> kernels;
    std::vector<uint32_t> args;
    std::unordered_map<std::string, size_t> shared_memory;

    // nullptr (with *err filled) on a missing file, malformed json, missing keys or an index
    // outside the storage table — the reference asserts or crashes on those.
    static Model* from_json(const char* json_file, std::string* err = nullptr);
    // 0 for an unknown stype (the reference asserts).
    static size_t get_stype_size(const std::string& stype);
};

class KernelProfile {
public:
    std::vector<int> latency;   // duration of one persistent wave at occupancy j+1
    int total_latency = 0;
};

class ModelProfile {
public:
    int model_latency = 0;
    // 1000 = microseconds as the reference wrote them; the profiler here writes nanoseconds
    // ("latency_unit_ns": 1) because B200 kernels run for a few microseconds.
    int latency_unit_ns = 1000;
    std::unordered_map<std::string, KernelProfile> kernel_latency;
    std::string to_json() const;
    static ModelProfile* from_json(const char* json_file, std::string* err = nullptr);
};

// View of one named blob inside a mapped .param file.
struct ParamBlob {
    const float* data;
    size_t count;
};

// .param = "TVM_MODEL_PARAMS\0" | u64 count | count x { key NUL | u64 n | n x f32 LE }
// (reference writer: script/tvm_generate_model.py:66-76; reader: model.cpp:82-121).  The file is
// memory-mapped and blobs are views into the mapping: no intermediate std::vector copies.
class ModelParam {
public:
    ~ModelParam();
    std::unordered_map<std::string, ParamBlob> blobs;
    size_t size() const { return blobs.size(); }
    const ParamBlob* find(const std::string& key) const;
private:
    friend class ModelParamParser;
    void* map_ = nullptr;
    size_t map_len_ = 0;
};

class ModelParamParser {
public:
    static ModelParam* parse_from_file(const char* param_file, std::string* err = nullptr);
};

}  // namespace executor
}  // namespace reef
