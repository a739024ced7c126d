// Internal declarations shared by the translation units of libw4a16_b200.so.
#pragma once
#include <cuda_runtime.h>

#include <cstdint>

#include "layout.cuh"

namespace w4 {

// ---- repack.cu -------------------------------------------------------------------------------
// glu_f > 0: the tiles interleave the gate and up row blocks of every expert (layout.cuh), glu_f = ffn / 16
void launch_repack_q(const uint32_t* q_orig, uint32_t* qt, int n, int k, int glu_f, cudaStream_t st);
// Biased-exponent range of the non-zero bf16 scales: range2[0] = min (preset 255), range2[1] = max (preset 0).
void launch_scale_range(const uint16_t* s_orig, size_t total, int* range2, cudaStream_t st);
// `group` is the group size of the TILED array; a source group covers `src_div` tiled groups.  bf16 scales are
// multiplied by 2^shift and stored as f16; err_flag (device int, may be null) is set to 1 if one of them is not
// exactly representable.
void launch_repack_s(const uint16_t* s_orig, uint16_t* stl, int n, int k, int group, int src_div, int scale_bf16,
                     int shift, int* err_flag, int glu_f, cudaStream_t st);
// the same for a chunk of source rows [16*rb0, 16*(rb0+nrbc)) (streamed uploads)
void launch_repack_q_rows(const uint32_t* q_chunk, uint32_t* qt, int n, int k, int rb0, int nrbc, int glu_f,
                          cudaStream_t st);
void launch_repack_s_rows(const uint16_t* s_chunk, uint16_t* stl, int n, int k, int group, int src_div, int scale_bf16,
                          int shift, int* err_flag, int rb0, int nrbc, int glu_f, cudaStream_t st);
void launch_unpack_q(const uint32_t* qt, uint32_t* q_orig, int n, int k, cudaStream_t st);
void launch_unpack_s(const uint16_t* stl, uint16_t* s_orig, int n, int k, int group, int src_div, cudaStream_t st);
// out: f32 [n][k] (out_f16 == 0) or f16 [n][k] (out_f16 == 1, round-to-nearest-even of the f32 value);
// out_mul: the power of two that undoes the shift of bf16 scales (1 otherwise)
void launch_dequant(const uint32_t* qt, const uint16_t* stl, void* out, int n, int k, int group,
                    int out_f16, float out_mul, cudaStream_t st);

// lane-order mirror of the CPU dot (parity gates): out f32 [t][n], x16 f16 [t][k]
void launch_lane_mirror(const uint32_t* qt, const uint16_t* stl, const void* x16, float* out, int n, int k, int group,
                        int t, float out_mul, cudaStream_t st);
void launch_cast_f16(const float* x, void* y16, size_t total, cudaStream_t st);

// ---- gemv.cu ---------------------------------------------------------------------------------
constexpr int GEMV_MAX_SEG = 4;
constexpr int GEMV_MAX_M = 8;

// Row-parallel tensor parallelism: every rank's receive areas, mapped into this device's address space (CUDA
// IPC).  world <= 1 disables the fused all-reduce.  A receive area holds, per launch parity and per source rank,
// that rank's partial sums [8 tokens][max_rows] f32; every word is the sentinel 0xffffffff until its source has
// written it, and the reader puts the sentinel back.
constexpr int TP_MAX_WORLD = 8;
constexpr int TP_MAX_CTAS = 64;   // 256-row blocks per row-parallel linear (n <= 16384)
struct TpComm {
    int rank, world;
    int max_rows;                     // rows per token of an area
    int area_floats;                  // floats per (parity, source) area = max_rows * 8
    float* buf[TP_MAX_WORLD];         // rank p's receive areas: [2 parities][world sources][8][max_rows] f32
    unsigned* seq;                    // local: number of fused launches completed
    unsigned* done;                   // local: row blocks that finished the current launch's exchange
    long long wait_cycles;            // limit of the wait for the peers' words (2^31 cycles, about a second, by default)
};

constexpr int DBG_LAUNCHES = 64;   // launches kept by the diagnostic timeline (slot = launch number mod 64)
constexpr int DBG_CTAS = 384;      // CTAs stamped per launch
constexpr int DBG_STAMPS = 16;     // stamps per CTA and launch

struct GemvSeg {
    const uint4* qt;
    const uint32_t* st;  // scale pairs, one u32 = (row j, row j+8)
    void* out;           // [m][n] f32 or f16
    int n;               // rows of this segment
    int cta0;            // first grid.x index of this segment
    float out_mul;       // power of two applied to the sums (undoes the shift of bf16 scales; normally 1)
};

struct GemvArgs {
    GemvSeg seg[GEMV_MAX_SEG];
    int nseg;
    int k;
    int group;
    int m;
    int out_f16;
    int ksplit;
    const uint16_t* x;  // f16 [m][k]
    float* part;        // [ksplit][grid_x][256][GEMV_MAX_M] partial sums (ksplit > 1)
    unsigned* counters; // [grid_x], zero on entry, left zero on exit
    int subnormal;      // 1: feed raw nibbles as f16 subnormals and fix up per group (default); 0: exact nibble-8
    int cluster;        // 1: the K splits of a row block form a thread-block cluster and reduce through DSMEM
    int cons_warps;     // consumer warps per CTA: 8 (two row blocks each) or 16 (one each)
    int ring_stages;    // 2 KB chunks in flight per warp (2..4)
    long long* dbg;     // optional timeline buffer (diagnostic): [DBG_LAUNCHES][DBG_CTAS][DBG_STAMPS] wall-clock stamps
    int dbg_seq;        // launch slot in that buffer
    int pdl;            // 1: launch with programmatic stream serialization (overlaps the previous kernel's tail)
    // grouped (MoE decode) mode: blockIdx.x / ctas_per_seg indexes a device table of <=8-row segments; the
    // single segment seg[0] then describes the stacked expert matrix (n = rows per expert)
    int grouped;
    int ctas_per_seg;
    int expert0;
    const int* tile_expert;
    const int* tile_row0;
    const int* tile_rows;
    const int* num_tiles;
    const float* row_w;   // optional factor per sorted row, applied at the final store
    int glu;              // 1: the rows are interleaved gate / up 16-row blocks (layout.cuh) and the kernel stores
                          // f16(silu(f16 gate) * f16 up), n/2 values per token, instead of the n sums
    const int* x_slot_of_pos;   // optional gather: sorted row r reads x row x_slot_of_pos[r] / x_slots_per_token
    int x_slots_per_token;
    int tables_fresh;     // 1: the launch just before this one wrote the segment table, so the table is read only after the
                          // dependency wait (with 0 the weights of the segment are requested while that kernel still drains)
    int rb_no_units;           // row-block form: 1 = never the 16-warp variant (tuning)
    int rb_stash, rb_stash2;   // row-block form, 16-warp variant: byte offsets of the weight slab and of the scale words in
                               // dynamic shared memory (set by the launcher)
    int nrb_w;            // 16-row blocks of the whole resident matrix (tile pitch); 0 = seg n / 16
    TpComm tp;          // fused all-reduce over peers (row-parallel); tp.world <= 1: off
    int* status;        // device word that records the first bounded wait that expired
};

// Total CTAs along x for the segments in `a` (fills seg[].cta0).
int gemv_plan_ctas(GemvArgs& a);
// Smallest and preferred split-K for a plan (see gemv.cu).
int gemv_pick_ksplit(int grid_x, int k, int group, int m, int sm_count, int max_split, int stages);
size_t gemv_smem_bytes(int k, int group, int m, int ksplit, int stages);
size_t gemv_part_floats(int grid_x, int ksplit);
cudaError_t launch_gemv(const GemvArgs& a, int grid_x, cudaStream_t st);
// Raises the dynamic shared-memory limit of the GEMV kernels on the current device.
cudaError_t gemv_init_device();

// ---- gemv_sk.cu: the persistent (two CTAs per SM, equal unit ranges) form of the decode GEMV ------
struct SkPlan {
    int units_per_row;  // 128-channel units (two k-blocks; the last may hold one) along K
    int rows;           // 256-row blocks over all segments
    long long units;    // rows * units_per_row
    int ctas;           // grid size; CTA p owns units [units*p/ctas, units*(p+1)/ctas)
    int nu_max;         // most units one CTA owns
    int x_stride;       // halves per staged token row (byte stride = 64 mod 128)
    int x_rows;         // token rows staged (m, plus one all-zero row when m < 8)
    int off_zc;         // f32 [local group][4 lane columns][4]: zero-point terms as MMA C operands
    int off_sc;         // u32 [16 row blocks][local group][8]: the CTA's scale pairs
    int off_ring;       // stages x 16 KB, 1024-byte aligned
    int off_bars;       // xbar, full[stages], empty[stages], scbar
    int stages;
    int prefetch;       // stages requested before griddepcontrol.wait (the rest right after it)
    int total;          // dynamic shared memory requested (at least 77 KB: never three CTAs on an SM)
};
SkPlan sk_make_plan(int k, int group, int m, int rows, int sm_count, int max_stages, int prefetch);
size_t sk_part_floats(const SkPlan& p);   // scratch for parked partial sums; counters: one per row block
cudaError_t launch_gemv_sk(const GemvArgs& a, const SkPlan& p, cudaStream_t st);
cudaError_t gemv_sk_init_device();
cudaError_t gemv_rb_init_device();
bool gemv_rb_fits(const GemvArgs& a);
int gemv_rb_plan(GemvArgs& a, int sm_count, int& rbw);
cudaError_t launch_gemv_rb(const GemvArgs& a, int total_units, int rbw, int sm_count, cudaStream_t st);
// The 16-warp variant of the row-block form takes this call (all units resident at once, shared memory fits).
bool gemv_ru_fits(const GemvArgs& a, int sm_count);
// Name of the kernel that launch_gemv_rb runs for this call.
const char* gemv_rb_variant(const GemvArgs& a, int total_units, int rbw, int sm_count);

// ---- gemm_tc.cu ------------------------------------------------------------------------------
// Raises the dynamic shared-memory limit of the tensor-core GEMM kernels on the current device.
cudaError_t gemm_init_device();
cudaError_t head_init_device();

// ---- moe.cu ----------------------------------------------------------------------------------
struct MoeBufs;
void launch_moe_topk(const float* logits, int* idx, float* wt, int t, int n_exp, int k, cudaStream_t st);
// histogram -> offsets + m-tile table (tiles of `bm` rows) -> placement of the local experts' slots
void launch_moe_align(const MoeBufs& b, int ns, int n_exp, int e0, int e1, int bm, cudaStream_t st);
// the same tables as topk + align for at most 1024 slots, in one launch of one block
int launch_moe_route_small(const float* logits, const MoeBufs& b, int t, int n_exp, int k, int e0, int e1, int bm,
                            cudaStream_t st);
void launch_moe_gather(const void* x, const MoeBufs& b, int ns, int k, int h, cudaStream_t st);
void launch_moe_act(const MoeBufs& b, int rows_upper, int ffn, cudaStream_t st);
void launch_moe_combine(const MoeBufs& b, void* out, int t, int h, int k, int out_f16, cudaStream_t st);

}  // namespace w4
