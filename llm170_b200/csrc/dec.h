// The decoder object behind the C ABI (one per device).
#pragma once
#include <map>
#include <string>
#include <vector>

#include "../../include/w4a16_b200.h"
#include "internal.h"

namespace w4 {

constexpr int DBG_SLOTS = DBG_LAUNCHES * DBG_CTAS * DBG_STAMPS;

struct Lin {
    uint32_t* qt = nullptr;  // T64 tiles (layout.cuh)
    uint16_t* st = nullptr;  // tiled f16 scale pairs
    int n = 0, k = 0, group = 0;   // group: of the resident scale tiles (128 or 32)
    int group_src = 0;             // group of the uploaded scales (64 is stored as two groups of 32)
    float out_mul = 1.0f;          // 2^-shift when bf16 scales had to be shifted into the f16 range (else 1)
    int glu_f = 0;                 // > 0: gate / up row blocks of every expert interleaved (layout.cuh), = ffn / 16
    size_t bytes = 0;
};

// MoE configuration (crates/backend-gpu/src/rawcuda/w4a16_dec/upload.rs:795-812) and device scratch.
struct MoeCfg {
    bool set = false;
    int n_experts = 0, top_k = 0, ffn = 0, hidden = 0, group = 32;
    int e0 = 0, e1 = 0;  // experts [e0, e1) are resident on this decoder (expert parallelism)
};

struct MoeBufs {
    int* idx = nullptr;          // [slots] expert of each (token, j) slot
    float* wt = nullptr;         // [slots] routing weight
    int *cnt = nullptr, *off = nullptr, *cursor = nullptr;  // [n_experts]
    int *pos_of_slot = nullptr, *slot_of_pos = nullptr;     // [slots]
    int *tile_expert = nullptr, *tile_row0 = nullptr, *tile_rows = nullptr;  // [max_tiles]
    int *n_tiles = nullptr, *n_rows = nullptr;
    float* row_w = nullptr;      // [slots] routing weight in sorted order
    void *xs = nullptr, *c13 = nullptr, *act = nullptr, *c2 = nullptr;  // f16 [slots][h | 2f | f | h]
    size_t cap_tokens = 0;
    int max_tiles = 0;
};

// The form of the decode GEMV chosen for a call (Dec::gemv_select).
struct GemvChoice {
    enum Form { PERSISTENT, SPLIT, ROWBLOCK } form = SPLIT;
    SkPlan sk{};
    int grid_x = 0;            // 256-row blocks over all segments (16-row blocks in the row-block form)
    size_t part_floats = 0;    // partial-sum scratch the launch needs
    size_t tickets = 0;        // arrival tickets the launch needs
    int rbw = 2;               // row-block form: 16-row blocks per CTA unit
    char name[64] = {0};       // the kernel instantiation, for reports
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
    std::vector<void*> retired;   // scratch blocks superseded by larger ones: freed with the decoder (graphs may hold them)
    int* err_flag = nullptr;       // device int[4]: repack error flag, bf16 exponent range (min, max)
    int* gemm_status = nullptr;  // device word: first bounded wait that expired in any kernel (0 = none)
    // device staging for the host-buffer entry points
    void* xh = nullptr;
    size_t xh_cap = 0;
    void* yh = nullptr;
    size_t yh_cap = 0;
    void* pin = nullptr;         // pinned host ring (two slots) and its device twin for streamed uploads / cache reads
    void* stage_dev = nullptr;
    size_t pin_cap = 0;
    void* x16 = nullptr;         // f16 copy of f32 activations (w4a16_lin_forward_x32)
    size_t x16_cap = 0;
    // int8 lm-head (head.cu): offset-binary bytes [n][k], f32 row scales
    uint8_t* head_q = nullptr;
    float* head_scale = nullptr;
    int head_n = 0, head_k = 0;
    // knobs
    int tune_gemv_stages = 4;
    int tune_gemv_rowblock_units = 1;  // 1: launches whose 32-row units are all resident at once run the 16-warp variant
    int tune_gemv_warps = 8;
    int tune_gemv_sk_stages = 4;   // most 16 KB ring stages of the persistent GEMV (2..6; fewer when x needs the room)
    int tune_gemv_sk_prefetch = 2; // ring stages the persistent GEMV requests before the previous kernel is complete
    int tune_gemv_rowblock = 1;    // up to four tokens of a g128 linear run one small CTA per 16-row block (gemv_rb.cu)
    int tune_gemv_persistent = 1;  // dense decode GEMV as two persistent CTAs per SM with equal unit ranges (gemv_sk.cu)
    int tune_gemv_cluster = 1;   // K splits of a row block as a thread-block cluster (DSMEM reduce) when 2 <= ksplit <= 8
    int tune_gemv_subnormal = 1;
    int tune_pdl = 1;
    int tune_tp_wait_log2 = 31;  // the fused all-reduce gives up on its peers after 2^this cycles
    int tune_gemm_mt = 0;        // 128-token blocks per GEMM tile: 0 = automatic, 1 or 2
    int tune_gemm_ksplit = 0;    // K splits of the GEMM: 0 = automatic (only when the tiles do not fill the SMs)
    int tune_gemm_tma_store = 1; // dense whole tiles leave through shared memory and TMA stores (0: per-lane stores)
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
    int upload_stream(const char* name, int n, int k, int group, int scale_bf16, w4a16_fill_fn fill, void* user,
                      int glu_f = 0);
    int upload_common(const char* name, const void* q_dev, const void* s_dev, int n, int k, int group,
                      int scale_bf16, int glu_f = 0);
    std::string last_kernel;   // instantiation launched by the last forward call
    int gemv_select(GemvArgs& a, bool allreduce, bool own_scratch, GemvChoice& c);
    int gemv_run(GemvArgs& a, const GemvChoice& c, cudaStream_t st);
    int gemv(const Lin* const* ls, int nseg, const void* x, void* const* outs, int t, int out_kind,
             cudaStream_t st, bool allreduce = false);
    int gemm(const Lin* l, const void* x, void* dst, int t, int out_kind, cudaStream_t st);
    int gemm_grouped(const Lin* l, const void* xs, int xs_rows, void* out, int n_per_expert, const MoeBufs& b,
                     int max_tiles, int mt, const float* row_w, cudaStream_t st);
    // row-parallel tensor parallelism (fused all-reduce in the GEMV): local exchange block + peer mappings
    TpComm tp{};
    void* tp_block = nullptr;
    void* tp_peer[TP_MAX_WORLD] = {};
    int tp_max_rows = 0;
    int gemv_grouped(const Lin* l, const void* xs, void* out, int n_per_expert, const MoeBufs& b, int max_tiles,
                     int est_tiles, const float* row_w, cudaStream_t st, const int* x_slot_of_pos = nullptr,
                     int x_slots_per_token = 1, bool tables_fresh = false);
    MoeCfg moe;
    MoeBufs mb;
    int ensure_moe(int t, cudaStream_t st);
    void free_moe(bool retire = false);
    int moe_ffn(int layer, const float* logits, const void* x16, void* y, int t, int out_kind, cudaStream_t st);
};

}  // namespace w4

// The opaque handle of the C ABI.
struct w4a16_dec {
    w4::Dec d;
};
