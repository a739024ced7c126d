// Prefill W4A16 GEMM (tensor cores). Placeholder translation unit until the tcgen05 kernel lands.
#include "dec.h"

namespace w4 {

int Dec::gemm(const Lin*, const void*, void*, int t, int, cudaStream_t) {
    return fail("w4a16 gemm: t=%d > 8 is not available in this build", t);
}

}  // namespace w4
