// Specialised decode-attention kernel for the (G=16, S=2, d=8, D=128, 4 query heads per KV head)
// geometry.  Placeholder until the kernel lands: reports "not supported" so that the generic
// kernel serves every geometry.

#include "common.cuh"

namespace tacvq {

bool attn_gsrq_supported(int, int, int, int, int, int) { return false; }
size_t attn_gsrq_workspace_bytes(int, int, int, int, int) { return 0; }
int attn_gsrq_dispatch(const __half *, const uint8_t *, const uint8_t *, const __half *, const __half *,
                       const int32_t *, const int32_t *, void *, __half *, float *, int, int, int, int64_t, int,
                       cudaStream_t) {
    return TACVQ_ERR_UNSUPPORTED;
}

}  // namespace tacvq
