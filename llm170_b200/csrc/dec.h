// The decoder object behind the C ABI (one per device).
#pragma once
#include <map>
#include <string>

#include "internal.h"

namespace w4 {

constexpr int DBG_SLOTS = 8192;

struct Lin {
    uint32_t* qt = nullptr;  // T64 tiles (layout.cuh)
    uint16_t* st = nullptr;  // tiled f16 scale pairs
    int n = 0, k = 0, group = 0;
    size_t bytes = 0;
};

struct Dec {
    int device = 0;
    int sm_count = 148;
    cudaStream_t stream = nullptr;
    std::map<std::string, Lin> lins;
    size_t weights_bytes = 0;
    // split-K scratch: partial sums and arrival tickets (zero between launches)
    float* part = nullptr;
    size_t part_cap = 0;
    unsigned* counters = nullptr;
    size_t counters_cap = 0;
    int* err_flag = nullptr;
    int* gemm_status = nullptr;  // device word: first bounded wait that expired in any kernel (0 = none)
    // device staging for the host-buffer entry points
    void* xh = nullptr;
    size_t xh_cap = 0;
    void* yh = nullptr;
    size_t yh_cap = 0;
    // knobs
    int tune_gemv_stages = 4;
    int tune_gemv_warps = 16;
    int tune_gemv_ctas_per_sm = 3;   // residency cap assumed by the split-K cost model (register-limited)
    int tune_gemv_subnormal = 1;
    int tune_pdl = 1;
    long long* dbg_buf = nullptr;  // device timeline buffer (DBG_SLOTS entries) when the knob is on
    int tune_gemv_ksplit = 0;
    // kernels launched by forward calls since creation
    unsigned long long launches = 0;
    std::string err;

    int fail(const char* fmt, ...);
    int cuda_fail(const char* what, cudaError_t e);
    static bool capturing(cudaStream_t st);
    int ensure_scratch(size_t part_floats, int grid_x, cudaStream_t st);
    void free_lin(Lin& l);
    int upload_common(const char* name, const void* q_dev, const void* s_dev, int n, int k, int group,
                      int scale_bf16);
    int gemv(const Lin* const* ls, int nseg, const void* x, void* const* outs, int t, int out_kind,
             cudaStream_t st);
    int gemm(const Lin* l, const void* x, void* dst, int t, int out_kind, cudaStream_t st);
};

}  // namespace w4
