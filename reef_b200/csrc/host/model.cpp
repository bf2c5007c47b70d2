#include "model.h"

#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <cstring>
#include <sstream>

#include "json.h"

namespace reef {

void log_error(const char* what, const char* file, int line) {
    if (getenv("REEF_QUIET") == nullptr) fprintf(stderr, "[reef] %s error, %s:%d\n", what, file, line);
}

namespace executor {

using util::JsonValue;

static bool set_err(std::string* err, const std::string& m) {
    if (err) *err = m;
    return false;
}

static bool get_uint(const JsonValue* v, uint64_t* out) {
    if (!v || !v->is(JsonValue::Number) || v->num < 0) return false;
    *out = (uint64_t)v->num;
    return true;
}

Model* Model::from_json(const char* json_file, std::string* err) {
    JsonValue root;
    std::string perr;
    if (!util::json_parse_file(json_file, &root, &perr)) {
        set_err(err, perr);
        return nullptr;
    }
    const JsonValue* jstorage = root.find("storage");
    const JsonValue* jkernels = root.find("kernels");
    const JsonValue* jargs = root.find("args");
    const JsonValue* jsmem = root.find("shared_memory");
    if (!jstorage || !jstorage->is(JsonValue::Array) || !jkernels || !jkernels->is(JsonValue::Array)) {
        set_err(err, "model json needs \"storage\" and \"kernels\" arrays");
        return nullptr;
    }
    std::unique_ptr<Model> m(new Model);
    for (auto& s : jstorage->arr) {
        const JsonValue* n = s.find("name");
        const JsonValue* st = s.find("stype");
        uint64_t size = 0;
        if (!n || !n->is(JsonValue::String) || !st || !st->is(JsonValue::String) || !get_uint(s.find("size"), &size)) {
            set_err(err, "malformed storage entry");
            return nullptr;
        }
        if (get_stype_size(st->str) == 0) {
            set_err(err, "unknown stype " + st->str);
            return nullptr;
        }
        m->storage.push_back(StorageInfo{n->str, (size_t)size, st->str});
    }
    for (auto& k : jkernels->arr) {
        KernelInfo ki;
        const JsonValue* n = k.find("name");
        const JsonValue* lp = k.find("launch_params");
        const JsonValue* ka = k.find("args");
        if (!n || !n->is(JsonValue::String) || !lp || !lp->is(JsonValue::Array) || lp->arr.size() != 6 || !ka ||
            !ka->is(JsonValue::Array)) {
            set_err(err, "malformed kernel entry");
            return nullptr;
        }
        ki.name = n->str;
        for (int i = 0; i < 6; i++) {
            uint64_t v;
            if (!get_uint(&lp->arr[i], &v)) {
                set_err(err, "bad launch_params in " + ki.name);
                return nullptr;
            }
            ki.launch_params[i] = (uint32_t)v;
        }
        for (auto& a : ka->arr) {
            uint64_t v;
            if (!get_uint(&a, &v) || v >= m->storage.size()) {
                set_err(err, "kernel " + ki.name + " names a storage index outside the table");
                return nullptr;
            }
            ki.args.push_back((size_t)v);
        }
        m->kernels.push_back(std::move(ki));
    }
    if (jargs && jargs->is(JsonValue::Array))
        for (auto& a : jargs->arr) {
            uint64_t v;
            if (!get_uint(&a, &v) || v >= m->storage.size()) {
                set_err(err, "\"args\" names a storage index outside the table");
                return nullptr;
            }
            m->args.push_back((uint32_t)v);
        }
    if (jsmem && jsmem->is(JsonValue::Object))
        for (auto& kv : jsmem->obj) {
            uint64_t v;
            if (!get_uint(&kv.second, &v)) {
                set_err(err, "bad shared_memory entry " + kv.first);
                return nullptr;
            }
            m->shared_memory[kv.first] = (size_t)v;
        }
    return m.release();
}

size_t Model::get_stype_size(const std::string& stype) {
    if (stype == "float32") return 4;
    if (stype == "int64") return 8;
    if (stype == "byte") return 1;
    if (stype == "uint1") return 1;
    if (stype == "int32") return 4;
    return 0;
}

ModelProfile* ModelProfile::from_json(const char* json_file, std::string* err) {
    JsonValue root;
    std::string perr;
    if (!util::json_parse_file(json_file, &root, &perr)) {
        set_err(err, perr);
        return nullptr;
    }
    uint64_t ml = 0;
    const JsonValue* kl = root.find("kernel_latency");
    if (!get_uint(root.find("model_latency"), &ml) || !kl || !kl->is(JsonValue::Object)) {
        set_err(err, "profile json needs model_latency and kernel_latency");
        return nullptr;
    }
    std::unique_ptr<ModelProfile> p(new ModelProfile);
    p->model_latency = (int)ml;
    uint64_t unit = 0;
    if (get_uint(root.find("latency_unit_ns"), &unit) && unit > 0) p->latency_unit_ns = (int)unit;
    for (auto& kv : kl->obj) {
        KernelProfile kp;
        uint64_t tl = 0;
        const JsonValue* lat = kv.second.find("latency");
        if (!get_uint(kv.second.find("total_latency"), &tl) || !lat || !lat->is(JsonValue::Array)) {
            set_err(err, "malformed profile of " + kv.first);
            return nullptr;
        }
        kp.total_latency = (int)tl;
        for (auto& v : lat->arr) kp.latency.push_back((int)v.num);
        p->kernel_latency.insert({kv.first, kp});
    }
    return p.release();
}

std::string ModelProfile::to_json() const {
    std::ostringstream ss;
    ss << "{\"model_latency\":" << model_latency;
    if (latency_unit_ns != 1000) ss << ",\"latency_unit_ns\":" << latency_unit_ns;
    ss << ",\"kernel_latency\":{";
    size_t i = 0;
    for (auto& pair : kernel_latency) {
        ss << "\"" << pair.first << "\":{\"total_latency\":" << pair.second.total_latency << ", \"latency\":[";
        for (size_t j = 0; j < pair.second.latency.size(); j++) {
            ss << pair.second.latency[j];
            if (j + 1 != pair.second.latency.size()) ss << ",";
        }
        ss << "]}";
        if (++i != kernel_latency.size()) ss << ",";
    }
    ss << "}}";
    return ss.str();
}

static const char kParamMagic[] = "TVM_MODEL_PARAMS";   // sizeof includes the NUL, 17 bytes

ModelParam::~ModelParam() {
    if (map_) munmap(map_, map_len_);
}

const ParamBlob* ModelParam::find(const std::string& key) const {
    auto it = blobs.find(key);
    return it == blobs.end() ? nullptr : &it->second;
}

ModelParam* ModelParamParser::parse_from_file(const char* param_file, std::string* err) {
    int fd = open(param_file, O_RDONLY);
    if (fd < 0) {
        set_err(err, std::string("cannot open ") + param_file);
        return nullptr;
    }
    struct stat st;
    if (fstat(fd, &st) != 0 || st.st_size < (off_t)(sizeof(kParamMagic) + 8)) {
        close(fd);
        set_err(err, "param file too short");
        return nullptr;
    }
    size_t len = (size_t)st.st_size;
    void* map = mmap(nullptr, len, PROT_READ, MAP_PRIVATE, fd, 0);
    close(fd);
    if (map == MAP_FAILED) {
        set_err(err, "mmap failed");
        return nullptr;
    }
    std::unique_ptr<ModelParam> p(new ModelParam);
    p->map_ = map;
    p->map_len_ = len;
    const unsigned char* b = (const unsigned char*)map;
    size_t off = 0;
    if (memcmp(b, kParamMagic, sizeof(kParamMagic)) != 0) {
        set_err(err, "bad .param magic");
        return nullptr;
    }
    off += sizeof(kParamMagic);
    uint64_t count;
    memcpy(&count, b + off, 8);
    off += 8;
    if (count == 0) {
        set_err(err, "empty .param");
        return nullptr;
    }
    for (uint64_t i = 0; i < count; i++) {
        const void* nul = off < len ? memchr(b + off, 0, len - off) : nullptr;
        if (!nul) {
            set_err(err, "truncated .param key");
            return nullptr;
        }
        std::string key((const char*)(b + off));
        off = (size_t)((const unsigned char*)nul - b) + 1;
        if (key.size() >= 256 || off + 8 > len) {   // the reference reads keys into a 256-byte buffer
            set_err(err, "bad .param key");
            return nullptr;
        }
        uint64_t n;
        memcpy(&n, b + off, 8);
        off += 8;
        if (n == 0 || n > (len - off) / 4) {
            set_err(err, "truncated .param array " + key);
            return nullptr;
        }
        p->blobs[key] = ParamBlob{(const float*)(b + off), (size_t)n};   // may be unaligned: only memcpy'd
        off += 4 * (size_t)n;
    }
    return p.release();
}

}  // namespace executor
}  // namespace reef
