// MoE routing, dispatch and combine around the grouped W4A16 GEMM.
//
// Follows the reference's resident-expert path (crates/backend-gpu/src/rawcuda/w4a16_dec/moe/mod.rs:263-447,
// crates/backend-gpu/src/rawcuda/w4a16_dec/kernels/marlin_moe.rs:290-422):
//   router top-k -> group the T*k (token, expert) slots by expert -> grouped GEMM-1 over gate|up ->
//   SiLU(gate)*up -> grouped GEMM-2 over down, scaled by the routing weight -> sum over k.
// Kernels here: top-k (crates/backend-gpu/src/rawcuda/assets/moe.cu:686-759), the expert histogram / offsets /
// placement that replace the single-block counting sort (crates/backend-gpu/src/rawcuda/assets/gptq4.cu:376-413,
// crates/backend-gpu/src/rawcuda/assets/moe.cu:1599-1633), the row gather, the activation
// (crates/backend-gpu/src/rawcuda/assets/moe.cu:1649-1660) and the top-k sum (:1662-1674).
// Slots of one expert are placed with an atomic cursor, so their order inside an expert's segment is
// not fixed; every output row is computed independently and the final sum runs over k in index order,
// so results do not depend on that order.
#include <cuda_fp16.h>

#include "dec.h"

namespace w4 {

namespace {

constexpr int TOPK_WARPS = 8;

// One warp per token, experts dealt to lanes round-robin (expert e lives in lane e % 32, slot e / 32).
// Same arithmetic as select_topk / moe_topk of the reference (crates/core/src/qwen35/stages/moe.rs:8-31,
// crates/backend-gpu/src/rawcuda/w4a16_dec/mod.rs:168-185), in the same order: p_e = exp(l_e - max) / sum with the
// sum taken sequentially over e = 0..n-1, pick k times the largest remaining p (ties: lower index), weights =
// p / (sum of the picked p, added in pick order).  Ordering on the normalised p, not on the numerators, matters
// when two different numerators round to the same p.  exp is evaluated in double and rounded once, the closest
// a device routine gets to the host's expf.  A pick is two warp-wide integer reductions: positive floats order
// like their bit patterns, so the largest p is a max over u32 and the tie-break a min over the indices that hold it.
// `stage`: optional shared-memory row of n floats owned by this warp; with it the sequential sum is read back by one
// lane (independent loads, one dependent add each) instead of travelling through n dependent shuffles.
// SLOTS = experts per lane the instantiation can hold (n <= 32 * SLOTS): a compile-time bound keeps the lane's values in
// registers.
template <int SLOTS>
__device__ __forceinline__ void topk_of_token_n(const float* __restrict__ l, int* __restrict__ idx, float* __restrict__ wt,
                                                int n, int k, int lane, float* stage) {
    float mx = -INFINITY;
    for (int i = lane; i < n; i += 32) {
        mx = fmaxf(mx, l[i]);
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
    }
    float pv[SLOTS];
    const int cnt = (n - lane + 31) >> 5;   // experts lane, lane + 32, ... below n
#pragma unroll
    for (int j = 0; j < SLOTS; ++j) {
        pv[j] = j < cnt ? (float)exp((double)(l[lane + 32 * j] - mx)) : 0.f;
    }
    // sum in index order, the same on every lane: element e = 32*j + src comes from lane src, slot j
    float sum = 0.f;
    if (stage != nullptr) {
#pragma unroll
        for (int j = 0; j < SLOTS; ++j) {
            if (j < cnt) {
                stage[lane + 32 * j] = pv[j];
            }
        }
        __syncwarp();
        if (lane == 0) {
            for (int e = 0; e < n; ++e) {
                sum += stage[e];
            }
        }
        sum = __shfl_sync(0xffffffffu, sum, 0);
        __syncwarp();   // the row may be reused for the warp's next token
    } else {
        const int slots = (n + 31) >> 5;
#pragma unroll
        for (int j = 0; j < SLOTS; ++j) {
            if (j < slots) {
                const float mine_j = pv[j];
                const int live = min(32, n - 32 * j);
                for (int src = 0; src < live; ++src) {
                    sum += __shfl_sync(0xffffffffu, mine_j, src);
                }
            }
        }
    }
#pragma unroll
    for (int j = 0; j < SLOTS; ++j) {
        pv[j] = pv[j] / sum;
    }
    unsigned used = 0u;
    float wsum = 0.f;
    float mine = 0.f;  // lane r keeps the r-th picked p
    for (int r = 0; r < k; ++r) {
        unsigned best = 0u;   // bit pattern of the lane's largest remaining p (p >= 0: patterns order like values)
#pragma unroll
        for (int j = 0; j < SLOTS; ++j) {
            if (j < cnt && !(used & (1u << j))) {
                best = max(best, __float_as_uint(pv[j]));
            }
        }
        const unsigned top = __reduce_max_sync(0xffffffffu, best);
        unsigned cand = 0xffffffffu;   // lowest index on this lane that holds `top`
#pragma unroll
        for (int j = SLOTS - 1; j >= 0; --j) {
            if (j < cnt && !(used & (1u << j)) && __float_as_uint(pv[j]) == top) {
                cand = (unsigned)(lane + 32 * j);
            }
        }
        const int bi = (int)__reduce_min_sync(0xffffffffu, cand);
        if ((bi & 31) == lane) {
            used |= 1u << (bi >> 5);
        }
        if (lane == 0) {
            idx[r] = bi;
        }
        const float bv = __uint_as_float(top);
        if (lane == (r & 31)) {
            mine = bv;
        }
        wsum += bv;
    }
    if (lane < k) {
        wt[lane] = mine / wsum;
    }
}

__device__ __forceinline__ void topk_of_token(const float* __restrict__ l, int* __restrict__ idx, float* __restrict__ wt,
                                              int n, int k, int lane, float* stage = nullptr) {
    if (n <= 128) {
        topk_of_token_n<4>(l, idx, wt, n, k, lane, stage);
    } else if (n <= 256) {
        topk_of_token_n<8>(l, idx, wt, n, k, lane, stage);
    } else {
        topk_of_token_n<32>(l, idx, wt, n, k, lane, stage);
    }
}

__global__ void moe_topk_kernel(const float* __restrict__ lg, int* __restrict__ idx, float* __restrict__ wt, int t,
                                int n, int k, int stage_rows) {
    extern __shared__ float s_stage[];   // [warps][n] when the launch provides it
    const int w = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int ti = blockIdx.x * TOPK_WARPS + w;
    if (ti >= t) {
        return;
    }
    topk_of_token(lg + (size_t)ti * n, idx + (size_t)ti * k, wt + (size_t)ti * k, n, k, lane,
                  stage_rows ? s_stage + (size_t)w * n : nullptr);
}

// Decode-sized batches (at most 1024 (token, expert) slots): routing, histogram, offsets, tile table, placement
// and sorted routing weights in ONE block of 1024 threads -- the six launches they take otherwise cost more
// than the expert matmuls of a single token.  Same tables as the separate kernels below.
__global__ void __launch_bounds__(1024)
moe_route_small_kernel(const float* __restrict__ lg, int* __restrict__ idx, float* __restrict__ wt,
                       int* __restrict__ off, int* __restrict__ pos_of_slot, int* __restrict__ slot_of_pos,
                       int* __restrict__ tile_expert, int* __restrict__ tile_row0, int* __restrict__ tile_rows,
                       int* __restrict__ n_tiles, int* __restrict__ n_rows, float* __restrict__ row_w, int t, int n_exp,
                       int k, int e0, int e1, int bm, int stage_rows, int do_topk) {
    __shared__ int s_rows[1024], s_tiles[1024], s_off[1024], s_cursor[1024];
    extern __shared__ float s_stage[];   // [32 warps][n_exp] when the launch provides it
    const int tid = threadIdx.x, w = tid >> 5, lane = tid & 31;
    s_rows[tid] = 0;
    s_cursor[tid] = 0;
    if (do_topk) {   // a handful of tokens: routed here; more: routed by moe_topk_kernel on many SMs just before
        for (int ti = w; ti < t; ti += 32) {
            topk_of_token(lg + (size_t)ti * n_exp, idx + (size_t)ti * k, wt + (size_t)ti * k, n_exp, k, lane,
                          stage_rows ? s_stage + (size_t)w * n_exp : nullptr);
        }
    }
    __syncthreads();   // idx / wt of every token are visible to the block
    const int ns = t * k;
    int my_e = -1;
    if (tid < ns) {
        my_e = idx[tid];
        if (my_e >= e0 && my_e < e1) {
            atomicAdd(&s_rows[my_e], 1);
        } else {
            my_e = -1;
        }
    }
    __syncthreads();
    // inclusive scan of (rows, tiles) over the 1024 experts slots: shuffles inside a warp, then the 32 warp totals
    const int c = s_rows[tid];
    const int ct = (c + bm - 1) / bm;
    int vr = c, vt = ct;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
        const int r = __shfl_up_sync(0xffffffffu, vr, d), tt = __shfl_up_sync(0xffffffffu, vt, d);
        if (lane >= d) {
            vr += r;
            vt += tt;
        }
    }
    __syncthreads();          // every thread has read its s_rows entry
    if (lane == 31) {
        s_rows[w] = vr;       // warp totals reuse the first 32 entries
        s_tiles[w] = vt;
    }
    __syncthreads();
    if (w == 0) {
        int tr = s_rows[lane], tl = s_tiles[lane];
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            const int r = __shfl_up_sync(0xffffffffu, tr, d), tt = __shfl_up_sync(0xffffffffu, tl, d);
            if (lane >= d) {
                tr += r;
                tl += tt;
            }
        }
        s_rows[lane] = tr;    // inclusive totals of warps 0..lane
        s_tiles[lane] = tl;
    }
    __syncthreads();
    const int base_r = w > 0 ? s_rows[w - 1] : 0, base_t = w > 0 ? s_tiles[w - 1] : 0;
    const int row0 = base_r + vr - c, tile0 = base_t + vt - ct;
    const int total_rows = s_rows[31], total_tiles = s_tiles[31];
    s_off[tid] = row0;
    if (tid < n_exp) {
        off[tid] = row0;
    }
    for (int r = 0, i = tile0; r < c; r += bm, ++i) {
        tile_expert[i] = tid;
        tile_row0[i] = row0 + r;
        tile_rows[i] = min(bm, c - r);
    }
    if (tid == 1023) {
        *n_tiles = total_tiles;
        *n_rows = total_rows;
    }
    __syncthreads();
    if (tid < ns) {
        int pos = -1;
        if (my_e >= 0) {
            pos = s_off[my_e] + atomicAdd(&s_cursor[my_e], 1);
            slot_of_pos[pos] = tid;
            row_w[pos] = wt[tid];
        }
        pos_of_slot[tid] = pos;  // -1: the expert lives on another rank
    }
}

__global__ void moe_count_kernel(const int* __restrict__ idx, int* __restrict__ cnt, int ns, int e0, int e1) {
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < ns; i += gridDim.x * blockDim.x) {
        const int e = idx[i];
        if (e >= e0 && e < e1) {
            atomicAdd(cnt + e, 1);
        }
    }
}

// One block of 1024 threads (n_exp <= 1024): exclusive offsets of the local experts' segments and the m-tile
// table of the grouped GEMM, tile i -> (expert, first sorted row, valid rows), both by a shared-memory scan.
// Also clears the placement cursors.
__global__ void moe_offsets_kernel(const int* __restrict__ cnt, int* __restrict__ off, int* __restrict__ cursor,
                                   int* __restrict__ tile_expert, int* __restrict__ tile_row0,
                                   int* __restrict__ tile_rows, int* __restrict__ n_tiles, int* __restrict__ n_rows,
                                   int n_exp, int e0, int e1, int bm) {
    __shared__ int s_rows[1024], s_tiles[1024];
    const int e = threadIdx.x;
    const int c = (e >= e0 && e < e1) ? cnt[e] : 0;
    s_rows[e] = c;
    s_tiles[e] = (c + bm - 1) / bm;
    __syncthreads();
    for (int d = 1; d < 1024; d <<= 1) {   // inclusive Hillis-Steele scan of both arrays
        const int r = e >= d ? s_rows[e - d] : 0, t = e >= d ? s_tiles[e - d] : 0;
        __syncthreads();
        s_rows[e] += r;
        s_tiles[e] += t;
        __syncthreads();
    }
    const int row0 = s_rows[e] - c, tile0 = s_tiles[e] - (c + bm - 1) / bm;
    if (e < n_exp) {
        off[e] = row0;
        cursor[e] = 0;
    }
    for (int r = 0, i = tile0; r < c; r += bm, ++i) {
        tile_expert[i] = e;
        tile_row0[i] = row0 + r;
        tile_rows[i] = min(bm, c - r);
    }
    if (e == 1023) {
        *n_tiles = s_tiles[e];
        *n_rows = s_rows[e];
    }
}

// placement of the local experts' slots in sorted order, with the routing weight of each sorted row
// (grouped matmul 2 multiplies by it)
__global__ void moe_place_kernel(const int* __restrict__ idx, const float* __restrict__ wt, const int* __restrict__ off,
                                 int* __restrict__ cursor, int* __restrict__ pos_of_slot, int* __restrict__ slot_of_pos,
                                 float* __restrict__ row_w, int ns, int e0, int e1) {
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < ns; i += gridDim.x * blockDim.x) {
        const int e = idx[i];
        int pos = -1;
        if (e >= e0 && e < e1) {
            pos = off[e] + atomicAdd(cursor + e, 1);
            slot_of_pos[pos] = i;
            row_w[pos] = wt[i];
        }
        pos_of_slot[i] = pos;  // -1: the expert lives on another rank
    }
}

// xs[pos][:] = x[slot / k][:]  (f16 rows of h), 16 bytes per thread
__global__ void moe_gather_kernel(const uint4* __restrict__ x, uint4* __restrict__ xs, const int* __restrict__ pos_of_slot,
                                  int ns, int k, int h8) {
    const size_t total = (size_t)ns * h8;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const int slot = (int)(i / h8), c = (int)(i % h8);
        const int pos = pos_of_slot[slot];
        if (pos >= 0) {
            xs[(size_t)pos * h8 + c] = x[(size_t)(slot / k) * h8 + c];
        }
    }
}

// act[pos][c] = f16( silu(gate) * up ),  c13 = [rows][2*ffn] with gate in the first half; 8 outputs per thread
__global__ void moe_act_silu_kernel(const __half* __restrict__ c13, __half* __restrict__ act, const int* __restrict__ n_rows,
                                    int ffn) {
    const int f8 = ffn / 8;
    const size_t total = (size_t)(*n_rows) * f8;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const size_t r = i / f8, c = (i % f8) * 8;
        const uint4 gv = *reinterpret_cast<const uint4*>(c13 + r * 2 * ffn + c);
        const uint4 uv = *reinterpret_cast<const uint4*>(c13 + r * 2 * ffn + ffn + c);
        const __half2* gh = reinterpret_cast<const __half2*>(&gv);
        const __half2* uh = reinterpret_cast<const __half2*>(&uv);
        uint4 ov;
        __half2* oh = reinterpret_cast<__half2*>(&ov);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float2 g = __half22float2(gh[j]), u = __half22float2(uh[j]);
            oh[j] = __floats2half2_rn((g.x / (1.0f + expf(-g.x))) * u.x, (g.y / (1.0f + expf(-g.y))) * u.y);
        }
        *reinterpret_cast<uint4*>(act + r * ffn + c) = ov;
    }
}

// out[t][c] = sum_j c2[pos(t*k+j)][c]  (routing weights were applied in GEMM-2's epilogue); slots whose
// expert is not local contribute nothing
template <bool OUT_F16>
__global__ void moe_combine_kernel(const __half* __restrict__ c2, void* __restrict__ out, const int* __restrict__ pos_of_slot,
                                   int t, int h, int k) {
    const int h8 = h / 8;
    const size_t total = (size_t)t * h8;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const int r = (int)(i / h8), c = (int)(i % h8) * 8;
        float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        for (int j = 0; j < k; ++j) {
            const int pos = pos_of_slot[r * k + j];
            if (pos >= 0) {
                const uint4 v = *reinterpret_cast<const uint4*>(c2 + (size_t)pos * h + c);
                const __half2* vh = reinterpret_cast<const __half2*>(&v);
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    const float2 f = __half22float2(vh[q]);
                    acc[2 * q] += f.x;
                    acc[2 * q + 1] += f.y;
                }
            }
        }
        if (OUT_F16) {
            uint4 ov;
            __half2* oh = reinterpret_cast<__half2*>(&ov);
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                oh[q] = __floats2half2_rn(acc[2 * q], acc[2 * q + 1]);
            }
            *reinterpret_cast<uint4*>((__half*)out + (size_t)r * h + c) = ov;
        } else {
            float4* o = reinterpret_cast<float4*>((float*)out + (size_t)r * h + c);
            o[0] = make_float4(acc[0], acc[1], acc[2], acc[3]);
            o[1] = make_float4(acc[4], acc[5], acc[6], acc[7]);
        }
    }
}

inline int blocks_for(size_t total, int threads) {
    size_t b = (total + threads - 1) / threads;
    if (b > 148 * 16) {
        b = 148 * 16;
    }
    return b < 1 ? 1 : (int)b;
}

}  // namespace

void launch_moe_topk(const float* logits, int* idx, float* wt, int t, int n_exp, int k, cudaStream_t st) {
    const int stage = n_exp <= 512;   // 8 warps x 512 floats = 16 KB of shared memory at most
    moe_topk_kernel<<<(t + TOPK_WARPS - 1) / TOPK_WARPS, TOPK_WARPS * 32, stage ? TOPK_WARPS * n_exp * sizeof(float) : 0, st>>>(
        logits, idx, wt, t, n_exp, k, stage);
}

// Returns the number of launches.  Up to eight tokens are routed by the table block itself (one launch); above that
// one block's 32 warps would route two or more tokens each in turn (27 us at 64 tokens), so the routing runs on
// many SMs first and the block only builds the tables.
int launch_moe_route_small(const float* logits, const MoeBufs& b, int t, int n_exp, int k, int e0, int e1, int bm,
                           cudaStream_t st) {
    const int stage = n_exp <= 256;   // 32 warps x 256 floats = 32 KB beside the 16 KB of tables
    const int own_topk = t <= 8;
    if (!own_topk) {
        launch_moe_topk(logits, b.idx, b.wt, t, n_exp, k, st);
    }
    moe_route_small_kernel<<<1, 1024, (stage && own_topk) ? 32 * n_exp * sizeof(float) : 0, st>>>(
        logits, b.idx, b.wt, b.off, b.pos_of_slot, b.slot_of_pos, b.tile_expert, b.tile_row0, b.tile_rows, b.n_tiles, b.n_rows,
        b.row_w, t, n_exp, k, e0, e1, bm, stage, own_topk);
    return own_topk ? 1 : 2;
}

void launch_moe_align(const MoeBufs& b, int ns, int n_exp, int e0, int e1, int bm, cudaStream_t st) {
    cudaMemsetAsync(b.cnt, 0, (size_t)n_exp * sizeof(int), st);
    moe_count_kernel<<<blocks_for(ns, 256), 256, 0, st>>>(b.idx, b.cnt, ns, e0, e1);
    moe_offsets_kernel<<<1, 1024, 0, st>>>(b.cnt, b.off, b.cursor, b.tile_expert, b.tile_row0, b.tile_rows, b.n_tiles,
                                          b.n_rows, n_exp, e0, e1, bm);
    moe_place_kernel<<<blocks_for(ns, 256), 256, 0, st>>>(b.idx, b.wt, b.off, b.cursor, b.pos_of_slot, b.slot_of_pos, b.row_w,
                                                          ns, e0, e1);
}

void launch_moe_gather(const void* x, const MoeBufs& b, int ns, int k, int h, cudaStream_t st) {
    moe_gather_kernel<<<blocks_for((size_t)ns * (h / 8), 256), 256, 0, st>>>((const uint4*)x, (uint4*)b.xs, b.pos_of_slot,
                                                                           ns, k, h / 8);
}

void launch_moe_act(const MoeBufs& b, int rows_upper, int ffn, cudaStream_t st) {
    moe_act_silu_kernel<<<blocks_for((size_t)rows_upper * (ffn / 8), 256), 256, 0, st>>>((const __half*)b.c13, (__half*)b.act,
                                                                                 b.n_rows, ffn);
}

void launch_moe_combine(const MoeBufs& b, void* out, int t, int h, int k, int out_f16, cudaStream_t st) {
    const int g = blocks_for((size_t)t * (h / 8), 256);
    if (out_f16) {
        moe_combine_kernel<true><<<g, 256, 0, st>>>((const __half*)b.c2, out, b.pos_of_slot, t, h, k);
    } else {
        moe_combine_kernel<false><<<g, 256, 0, st>>>((const __half*)b.c2, out, b.pos_of_slot, t, h, k);
    }
}

}  // namespace w4
