// Host side of the tcgen05 attention kernel: tensor map over the fused QKV buffer, launch.
#include "attention_tc.cuh"

#include <cmath>
#include <cstring>
#include <string>

#include "registry.h"

namespace reef {

typedef CUresult (*att_encode_fn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static att_encode_fn g_att_encode = nullptr;

int att_smem_bytes() { return ATT_SMEM; }

int att_supported(int s, int heads, int d) { return (d == ATT_D && s >= 1 && s <= ATT_MAX_S && heads >= 1) ? 1 : 0; }

int att_build_params(int s, int heads, int has_mask, void* const* a, AttParams* P) {
    if (!g_att_encode) {
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult q;
        cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q);
        if (e != cudaSuccess || q != cudaDriverEntryPointSuccess || !fn) {
            set_error("cuTensorMapEncodeTiled is not available from the driver");
            return REEF_FAIL;
        }
        g_att_encode = (att_encode_fn)fn;
    }
    memset(P, 0, sizeof(*P));
    const int H = heads * ATT_D;
    P->qkv = (const float*)a[0];
    P->mask = has_mask ? (const float*)a[1] : nullptr;
    P->out = (float*)a[has_mask ? 2 : 1];
    P->S = s;
    P->heads = heads;
    P->scale = 1.0f / sqrtf((float)ATT_D);
    cuuint64_t dims[2] = {(cuuint64_t)(3 * H), (cuuint64_t)s};
    cuuint64_t strides[1] = {(cuuint64_t)(3 * H) * 4};
    cuuint32_t box[2] = {32, 128};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = g_att_encode(&P->tm_qkv, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<float*>(P->qkv), dims, strides, box, estr,
                              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        set_error("cuTensorMapEncodeTiled(attention) failed with CUresult " + std::to_string((int)r));
        return REEF_FAIL;
    }
    return tc_error_word(&P->error_word);
}

static bool g_att_attr_set[16] = {false};

int att_prepare_device() {
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 16 && !g_att_attr_set[dev]) {
        const void* fns[2] = {(const void*)reef_attention_tc_kernel<false>, (const void*)reef_attention_tc_kernel<true>};
        for (const void* fn : fns) {
            cudaError_t e = cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, ATT_SMEM);
            if (e == cudaSuccess)
                e = cudaFuncSetAttribute(fn, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
            if (e != cudaSuccess) {
                set_error(std::string("cudaFuncSetAttribute(attention_tc): ") + cudaGetErrorString(e));
                return REEF_FAIL;
            }
        }
        int* w = nullptr;
        int rc = tc_error_word(&w);
        if (rc != REEF_SUCC) return rc;
        g_att_attr_set[dev] = true;
    }
    return REEF_SUCC;
}

int att_launch(const AttParams& P0, cudaStream_t st, const int* flag, int* slot, int head_begin, int head_count) {
    AttParams P = P0;
    if (head_count < 0) head_count = P.heads - head_begin;
    if (head_begin < 0 || head_count <= 0 || head_begin + head_count > P.heads) {
        set_error("tensor-core attention: head range outside the kernel");
        return REEF_OUT_OF_RANGE;
    }
    P.preempt_flag = flag;
    P.task_slot = slot;
    P.head_begin = head_begin;
    P.stamps = flag != nullptr ? preempt_stamps_ptr() : nullptr;
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof(cfg));
    cfg.gridDim = dim3(head_count, 1, 1);
    cfg.blockDim = dim3(ATT_THREADS);
    cfg.dynamicSmemBytes = ATT_SMEM;
    cfg.stream = st;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr.val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    cudaError_t e = flag != nullptr ? cudaLaunchKernelEx(&cfg, reef_attention_tc_kernel<true>, P)
                                    : cudaLaunchKernelEx(&cfg, reef_attention_tc_kernel<false>, P);
    if (e != cudaSuccess) {
        set_error(std::string("cudaLaunchKernelEx(attention_tc): ") + cudaGetErrorString(e));
        return REEF_FAIL;
    }
    return REEF_SUCC;
}

int att_func_attrs(cudaFuncAttributes* fa, int* occ) {
    cudaError_t e = cudaFuncGetAttributes(fa, (const void*)reef_attention_tc_kernel<false>);
    if (e != cudaSuccess) {
        set_error(std::string("cudaFuncGetAttributes(attention_tc): ") + cudaGetErrorString(e));
        return REEF_FAIL;
    }
    *occ = 2;
    return REEF_SUCC;
}

}  // namespace reef
