// Decode-time W4A16 split-K GEMV for 1..8 tokens:  y[m][n] = sum_k x[m][k] * (q[n][k]-8) * s[n][k/group].
//
// Takes the place of the reference's split-K GEMV pair (crates/backend-gpu/src/rawcuda/assets/decode.cu:46-267,
// launched from crates/backend-gpu/src/rawcuda/w4a16_dec/kernels/decode.rs:23-127) and of its FFMA
// small-batch family (crates/backend-gpu/src/rawcuda/assets/gptq4.cu:44-723).  Differences by design:
//   * the 16 rows of each mma.sync m16n8k16 are WEIGHT rows and the 8 columns are tokens, so
//     m = 1..8 all use the same kernel and no MMA row is padding;
//   * weights never become rounded f16 values: the MMA multiplies the raw nibble (as an exact f16
//     subnormal, nibble * 2^-24 or 2^-20) by x, and the power of two, the zero point 8 (through a
//     per-group sum of x) and the f32 group scale are applied to the f32 accumulator once per group;
//   * each warp streams its row block through a private ring of 2 KB bulk (TMA) copies in shared
//     memory, so the bytes in flight do not depend on registers or occupancy;
//   * split-K partials are reduced by the last CTA to arrive (atomic ticket, no spin, fixed summation
//     order): no second launch, reproducible results, and the tickets are left at zero for graph replay.
// The kernel is HBM-bound: each lane consumes 16-byte pieces of the T64 layout (layout.cuh).
#include <cuda_fp16.h>

#include "internal.h"
#include "ptx.cuh"

namespace w4 {

namespace {

constexpr int MAX_RING_STAGES = 4;
constexpr int CHUNK_KB = 4;                         // k-blocks per bulk copy
constexpr int CHUNK_BYTES = CHUNK_KB * TILE_WORDS * 4;  // 2 KB
constexpr int ROWS_PER_CTA = GEMV_WARPS * TILE_ROWS;

__device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// first MMA of a group: accumulates onto zero
__device__ __forceinline__ void mma16816_z(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%10,%10,%10,%10};"
        : "=f"(c[0]), "=f"(c[1]), "=f"(c[2]), "=f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "f"(0.f));
}

// K range of split `s` in units of max(group, 64) input channels; ragged splits allowed.
__device__ __host__ __forceinline__ void split_range(int k, int group, int ksplit, int s, int* kb0, int* kb1) {
    const int unit_kb = group > TILE_K ? group / TILE_K : 1;
    const int units = k / (unit_kb * TILE_K);
    const int u0 = (int)(((long long)units * s) / ksplit);
    const int u1 = (int)(((long long)units * (s + 1)) / ksplit);
    *kb0 = u0 * unit_kb;
    *kb1 = u1 * unit_kb;
}

__host__ __forceinline__ int max_split_kblocks(int k, int group, int ksplit) {
    int mx = 0;
    for (int s = 0; s < ksplit; ++s) {
        int a, b;
        split_range(k, group, ksplit, s, &a, &b);
        mx = (b - a) > mx ? (b - a) : mx;
    }
    return mx;
}

struct SmemPlan {
    int x_stride;   // halves per token row (byte stride = 64 mod 128: conflict-free 128-bit reads)
    int x_rows;     // token rows staged (m, plus one all-zero row when m < 8)
    int off_xsum;   // f32 [groups][8]: -8 * sum of x over the group, per token
    int off_ring;   // GEMV_WARPS x RING_STAGES x CHUNK_BYTES
    int off_bars;   // 1 + GEMV_WARPS*stages mbarriers
    int stages;     // chunks in flight per warp
    int total;
};

__host__ SmemPlan make_plan(int k, int group, int m, int ksplit, int stages) {
    SmemPlan p;
    p.stages = stages < 2 ? 2 : (stages > MAX_RING_STAGES ? MAX_RING_STAGES : stages);
    const int halves = max_split_kblocks(k, group, ksplit) * TILE_K;
    p.x_stride = halves + 32;
    p.x_rows = m < GEMV_MAX_M ? m + 1 : m;
    int off = p.x_rows * p.x_stride * 2;
    off = (off + 127) & ~127;
    p.off_xsum = off;
    off += (halves / group) * GEMV_MAX_M * 4;
    off = (off + 127) & ~127;
    p.off_ring = off;
    off += GEMV_WARPS * p.stages * CHUNK_BYTES;
    p.off_bars = off;
    off += (1 + GEMV_WARPS * p.stages) * 8;
    p.total = off;
    return p;
}

template <int GROUP, bool SUBN>
__global__ void __launch_bounds__(GEMV_WARPS * 32)
gemv_w4a16_kernel(const GemvArgs a, const SmemPlan p) {
    extern __shared__ __align__(128) unsigned char smem[];
    __shared__ int s_is_last;
    __shared__ int s_abort;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int split = blockIdx.y;
    const int nkb = a.k / TILE_K;
    constexpr int KB_PER_GROUP = GROUP >= TILE_K ? GROUP / TILE_K : 1;   // 2 for g128, 1 for g32
    constexpr int GROUPS_PER_KB = GROUP >= TILE_K ? 1 : TILE_K / GROUP;  // 1 for g128, 2 for g32

    // segment of this CTA (q|k|v or gate|up share one launch, as in decode.cu:180-205)
    int si = 0;
#pragma unroll
    for (int i = 1; i < GEMV_MAX_SEG; ++i) {
        if (i < a.nseg && (int)blockIdx.x >= a.seg[i].cta0) {
            si = i;
        }
    }
    const GemvSeg& sg = a.seg[si];
    const int rb = ((int)blockIdx.x - sg.cta0) * GEMV_WARPS + warp;
    const bool warp_active = rb < sg.n / TILE_ROWS;

    int kb0, kb1;
    split_range(a.k, GROUP, a.ksplit, split, &kb0, &kb1);
    const int nloc = kb1 - kb0;                      // k-blocks of this split
    const int halves = nloc * TILE_K;
    const int ngl = halves / GROUP;                  // scale groups of this split

    const uint32_t sbase = smem_u32(smem);
    const uint32_t xbar = sbase + p.off_bars;
    const int RING_STAGES = p.stages;
    const uint32_t ring = sbase + p.off_ring + (uint32_t)warp * (RING_STAGES * CHUNK_BYTES);
    const uint32_t rbar = xbar + 8u + (uint32_t)warp * (RING_STAGES * 8);
    volatile int* abort_flag = &s_abort;

    if (threadIdx.x == 0) {
        s_abort = 0;
        mbar_init(xbar, 1);
        for (int i = 0; i < GEMV_WARPS * RING_STAGES; ++i) {
            mbar_init(xbar + 8u + 8u * i, 1);
        }
        mbar_init_fence();
    }
    // the all-zero token row read by MMA columns >= m
    if (a.m < GEMV_MAX_M) {
        uint4* z = reinterpret_cast<uint4*>(smem + (size_t)a.m * p.x_stride * 2);
        for (int i = threadIdx.x; i < p.x_stride / 8; i += blockDim.x) {
            z[i] = make_uint4(0, 0, 0, 0);
        }
    }
    __syncthreads();

    const int nchunks = (nloc + CHUNK_KB - 1) / CHUNK_KB;
    const unsigned char* wsrc =
        reinterpret_cast<const unsigned char*>(sg.qt) + ((size_t)(warp_active ? rb : 0) * nkb + kb0) * (TILE_WORDS * 4);
    auto issue_chunk = [&](int c) {
        const int kbs = min(CHUNK_KB, nloc - c * CHUNK_KB);
        const uint32_t bar = rbar + 8u * (c % RING_STAGES);
        mbar_expect_tx(bar, kbs * TILE_WORDS * 4);
        bulk_load(ring + (c % RING_STAGES) * CHUNK_BYTES, wsrc + (size_t)c * CHUNK_BYTES, kbs * TILE_WORDS * 4, bar);
    };
    if (warp_active && lane == 0) {
        for (int c = 0; c < RING_STAGES && c < nchunks; ++c) {
            issue_chunk(c);
        }
    }
    // Programmatic dependent launch: the weight copies above do not depend on the previous kernel in the
    // stream, so they are already in flight while it drains.  Everything below reads x or writes
    // scratch/outputs and must wait for it.  (Both instructions do nothing in an ordinary launch.)
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    if (threadIdx.x == 0) {
        mbar_expect_tx(xbar, a.m * halves * 2);
        for (int tok = 0; tok < a.m; ++tok) {
            bulk_load(sbase + tok * p.x_stride * 2, a.x + (size_t)tok * a.k + (size_t)kb0 * TILE_K, halves * 2, xbar);
        }
    }

    bool ok = mbar_wait(xbar, 0, abort_flag, a.status, (10 << 16));
    if (SUBN && ok) {
        // xsum[grp][tok] = -8 * sum_{k in grp} x[tok][k]   (tokens >= m: 0)
        float* xsum = reinterpret_cast<float*>(smem + p.off_xsum);
        for (int pr = warp; pr < ngl * GEMV_MAX_M; pr += GEMV_WARPS) {
            const int grp = pr >> 3, tok = pr & 7;
            float v = 0.f;
            if (tok < a.m) {
                const __half* xr = reinterpret_cast<const __half*>(smem) + (size_t)tok * p.x_stride + grp * GROUP;
                if (GROUP == 128) {
                    const uint2 u = *reinterpret_cast<const uint2*>(xr + lane * 4);
                    const float2 f0 = __half22float2(*reinterpret_cast<const __half2*>(&u.x));
                    const float2 f1 = __half22float2(*reinterpret_cast<const __half2*>(&u.y));
                    v = (f0.x + f0.y) + (f1.x + f1.y);
                } else {
                    v = __half2float(xr[lane]);
                }
            }
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) {
                v += __shfl_xor_sync(0xffffffffu, v, off);
            }
            if (lane == 0) {
                xsum[pr] = -8.f * v;
            }
        }
    }
    __syncthreads();

    float tot[4] = {0.f, 0.f, 0.f, 0.f};
    if (warp_active && ok) {
        const int ng = a.k / GROUP;
        const uint32_t* sp = sg.st + ((size_t)rb * ng + (size_t)kb0 * GROUPS_PER_KB / KB_PER_GROUP) * 8 + g;
        // B fragment source: token g (the zero row when g >= m), this lane's 8 k of each half k-block
        const int xrow_i = g < a.m ? g : a.m;
        uint32_t xaddr = sbase + (uint32_t)(xrow_i * p.x_stride + 8 * t) * 2;
        uint32_t xs_addr = sbase + p.off_xsum + (uint32_t)(2 * t) * 4;
        const uint32_t waddr = ring + lane * 16;

        float acc[4] = {0.f, 0.f, 0.f, 0.f}, acb[4] = {0.f, 0.f, 0.f, 0.f};  // two independent MMA chains
        uint32_t sc = __ldg(sp);
        int gl = 0;  // local group index

        auto finish_group = [&]() {
            const float2 sf = __half22float2(*reinterpret_cast<const __half2*>(&sc));
            ++gl;
            if (gl < ngl) {
                sc = __ldg(sp + (size_t)gl * 8);  // prefetch the next group's scales
            }
            acc[0] += acb[0];
            acc[1] += acb[1];
            acc[2] += acb[2];
            acc[3] += acb[3];
            if (SUBN) {
                const float2 z = lds_f32x2(xs_addr);
                xs_addr += GEMV_MAX_M * 4;
                tot[0] = fmaf(fmaf(acc[0], 16777216.f, z.x), sf.x, tot[0]);
                tot[1] = fmaf(fmaf(acc[1], 16777216.f, z.y), sf.x, tot[1]);
                tot[2] = fmaf(fmaf(acc[2], 1048576.f, z.x), sf.y, tot[2]);
                tot[3] = fmaf(fmaf(acc[3], 1048576.f, z.y), sf.y, tot[3]);
            } else {
                tot[0] = fmaf(acc[0], sf.x, tot[0]);
                tot[1] = fmaf(acc[1], sf.x, tot[1]);
                tot[2] = fmaf(acc[2], sf.y, tot[2]);
                tot[3] = fmaf(acc[3], sf.y, tot[3]);
            }
        };
        auto expand = [&](uint32_t w, uint32_t (&fr)[4]) {
            if (SUBN) {
                nibbles_as_subnormals(w, fr);
            } else {
                dequant_word(w, fr);
            }
        };
        // one k-block: 4 MMAs; `first` = this k-block starts a scale group (g128) -- g32 groups are half k-blocks
        auto kblock = [&](uint32_t wa, uint32_t xa, bool first, bool last) {
            const uint4 w = lds128(wa);
            const uint4 x0 = lds128(xa), x1 = lds128(xa + 64);
            uint32_t fr[4];
            expand(w.x, fr);
            if (first || GROUP < TILE_K) {
                mma16816_z(acc, fr, x0.x, x0.y);
            } else {
                mma16816(acc, fr, x0.x, x0.y);
            }
            expand(w.y, fr);
            if (first || GROUP < TILE_K) {
                mma16816_z(acb, fr, x0.z, x0.w);
            } else {
                mma16816(acb, fr, x0.z, x0.w);
            }
            if (GROUP < TILE_K) {
                finish_group();
            }
            expand(w.z, fr);
            if (GROUP < TILE_K) {
                mma16816_z(acc, fr, x1.x, x1.y);
            } else {
                mma16816(acc, fr, x1.x, x1.y);
            }
            expand(w.w, fr);
            if (GROUP < TILE_K) {
                mma16816_z(acb, fr, x1.z, x1.w);
            } else {
                mma16816(acb, fr, x1.z, x1.w);
            }
            if (GROUP < TILE_K || last) {
                finish_group();
            }
        };

        for (int c = 0; c < nchunks; ++c) {
            const int stg = c % RING_STAGES;
            ok = mbar_wait(rbar + 8u * stg, (c / RING_STAGES) & 1, abort_flag, a.status, (11 << 16) | c);
            if (!ok) {
                break;
            }
            const uint32_t wa = waddr + stg * CHUNK_BYTES;
            if (c * CHUNK_KB + CHUNK_KB <= nloc) {
                // group boundaries fall on even k-blocks: splits are whole groups
                kblock(wa, xaddr, true, KB_PER_GROUP == 1);
                kblock(wa + 512, xaddr + 128, KB_PER_GROUP == 1, true);
                kblock(wa + 1024, xaddr + 256, true, KB_PER_GROUP == 1);
                kblock(wa + 1536, xaddr + 384, KB_PER_GROUP == 1, true);
            } else {
                const int rem = nloc - c * CHUNK_KB;
                for (int i = 0; i < rem; ++i) {
                    const bool first = KB_PER_GROUP == 1 || (i & 1) == 0;
                    const bool last = KB_PER_GROUP == 1 || (i & 1) == 1;
                    kblock(wa + i * 512, xaddr + i * 128, first, last);
                }
            }
            xaddr += CHUNK_KB * 128;
            __syncwarp();
            if (lane == 0 && c + RING_STAGES < nchunks) {
                issue_chunk(c + RING_STAGES);
            }
        }
    }

    // tot[0],tot[1]: row g, tokens 2t, 2t+1 ; tot[2],tot[3]: row g+8, tokens 2t, 2t+1
    const int row0 = rb * TILE_ROWS + g, row1 = row0 + 8;
    if (a.ksplit == 1) {
        if (warp_active) {
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                const int tok = 2 * t + j;
                if (tok < a.m) {
                    if (a.out_f16) {
                        __half* o = reinterpret_cast<__half*>(sg.out) + (size_t)tok * sg.n;
                        o[row0] = __float2half_rn(tot[j]);
                        o[row1] = __float2half_rn(tot[2 + j]);
                    } else {
                        float* o = reinterpret_cast<float*>(sg.out) + (size_t)tok * sg.n;
                        o[row0] = tot[j];
                        o[row1] = tot[2 + j];
                    }
                }
            }
        }
        return;
    }

    // split-K: park partials as part[split][cta][row_in_cta (128)][tok (8)], then the last CTA of
    // this column of the grid sums the splits in index order.
    float* mypart = a.part + ((size_t)split * gridDim.x + blockIdx.x) * (ROWS_PER_CTA * GEMV_MAX_M);
    {
        const int lr0 = warp * TILE_ROWS + g, lr1 = lr0 + 8;
        *reinterpret_cast<float2*>(mypart + lr0 * GEMV_MAX_M + 2 * t) = make_float2(tot[0], tot[1]);
        *reinterpret_cast<float2*>(mypart + lr1 * GEMV_MAX_M + 2 * t) = make_float2(tot[2], tot[3]);
    }
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        const unsigned ticket = atomicAdd(a.counters + blockIdx.x, 1u);
        s_is_last = (ticket == (unsigned)a.ksplit - 1u);
    }
    __syncthreads();
    if (!s_is_last) {
        return;
    }
    __threadfence();
    const int nrows = min(ROWS_PER_CTA, sg.n - ((int)blockIdx.x - sg.cta0) * ROWS_PER_CTA);
    for (int i = threadIdx.x; i < ROWS_PER_CTA * (GEMV_MAX_M / 2); i += blockDim.x) {
        // one thread sums a (row, token pair): consecutive threads read consecutive float2
        const int lr = i / (GEMV_MAX_M / 2), tp = i % (GEMV_MAX_M / 2);
        if (lr < nrows && 2 * tp < a.m) {
            const float* src = a.part + (size_t)blockIdx.x * (ROWS_PER_CTA * GEMV_MAX_M) + lr * GEMV_MAX_M + 2 * tp;
            const size_t stride = (size_t)gridDim.x * (ROWS_PER_CTA * GEMV_MAX_M);
            float2 sum = make_float2(0.f, 0.f);
            for (int s = 0; s < a.ksplit; ++s) {
                const float2 v = __ldcg(reinterpret_cast<const float2*>(src + s * stride));
                sum.x += v.x;
                sum.y += v.y;
            }
            const int row = ((int)blockIdx.x - sg.cta0) * ROWS_PER_CTA + lr;
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                const int tok = 2 * tp + j;
                if (tok < a.m) {
                    const float v = j ? sum.y : sum.x;
                    if (a.out_f16) {
                        reinterpret_cast<__half*>(sg.out)[(size_t)tok * sg.n + row] = __float2half_rn(v);
                    } else {
                        reinterpret_cast<float*>(sg.out)[(size_t)tok * sg.n + row] = v;
                    }
                }
            }
        }
    }
    if (threadIdx.x == 0) {
        a.counters[blockIdx.x] = 0;  // ready for the next launch (graph replay needs no memset)
    }
}

constexpr int GEMV_SMEM_LIMIT = 112 * 1024;
constexpr int SM_SMEM_BYTES = 233472;  // 228 KB per SM, 1 KB reserved per resident CTA

}  // namespace

int gemv_plan_ctas(GemvArgs& a) {
    int ctas = 0;
    for (int i = 0; i < a.nseg; ++i) {
        a.seg[i].cta0 = ctas;
        const int nrb = a.seg[i].n / TILE_ROWS;
        ctas += (nrb + GEMV_WARPS - 1) / GEMV_WARPS;
    }
    return ctas;
}

size_t gemv_smem_bytes(int k, int group, int m, int ksplit, int stages) {
    return (size_t)make_plan(k, group, m, ksplit, stages).total;
}

size_t gemv_part_floats(int grid_x, int ksplit) {
    return ksplit > 1 ? (size_t)ksplit * grid_x * (ROWS_PER_CTA * GEMV_MAX_M) : 0;
}

// Split-K chosen by a small cost model instead of a fixed target (the reference sizes its split for a
// 70-SM part: crates/backend-gpu/src/rawcuda/w4a16_dec/kernels/decode.rs:3-20).  For every candidate the
// time is  waves x (largest split + fixed per-CTA cost), with all CTAs that fit resident at once sharing
// an SM's bandwidth; the cheapest wins, ties to fewer splits (fewer partials to reduce).
int gemv_pick_ksplit(int grid_x, int k, int group, int m, int sm_count, int max_ctas_per_sm, int stages) {
    const int unit = group > TILE_K ? group : TILE_K;
    const int units = k / unit;
    const double fixed = 3.0 * (128.0 / unit);  // per-CTA prologue + reduce, in units of work
    int best = 1;
    double best_cost = 1e30;
    for (int ks = 1; ks <= units && ks <= 64; ++ks) {
        const size_t smem = gemv_smem_bytes(k, group, m, ks, stages);
        if (smem > (size_t)GEMV_SMEM_LIMIT) {
            continue;
        }
        int ctas_per_sm = (int)(SM_SMEM_BYTES / (smem + 1024));
        if (ctas_per_sm > max_ctas_per_sm) {
            ctas_per_sm = max_ctas_per_sm;
        }
        const int per_split = (units + ks - 1) / ks;
        const long long ctas = (long long)grid_x * ks;
        const long long slots = (long long)sm_count * ctas_per_sm;
        const long long waves = (ctas + slots - 1) / slots;
        // CTAs on the busiest SM in the last wave
        const long long last = ctas - (waves - 1) * slots;
        const long long busiest = (last + sm_count - 1) / sm_count;
        const double cost = ((waves - 1) * ctas_per_sm + busiest) * (per_split + fixed);
        if (cost < best_cost * 0.999) {
            best_cost = cost;
            best = ks;
        }
    }
    return best;
}

cudaError_t gemv_init_device() {
    cudaError_t e;
#define W4_SET(K) \
    e = cudaFuncSetAttribute(K, cudaFuncAttributeMaxDynamicSharedMemorySize, GEMV_SMEM_LIMIT); \
    if (e != cudaSuccess) return e;
    W4_SET((gemv_w4a16_kernel<128, true>))
    W4_SET((gemv_w4a16_kernel<128, false>))
    W4_SET((gemv_w4a16_kernel<32, true>))
    W4_SET((gemv_w4a16_kernel<32, false>))
#undef W4_SET
    return cudaSuccess;
}

cudaError_t launch_gemv(const GemvArgs& a, int grid_x, cudaStream_t st) {
    const SmemPlan p = make_plan(a.k, a.group, a.m, a.ksplit, a.ring_stages);
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(grid_x, a.ksplit);
    cfg.blockDim = dim3(GEMV_WARPS * 32);
    cfg.dynamicSmemBytes = p.total;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = a.pdl ? 1 : 0;
    if (a.group == 128) {
        if (a.subnormal) {
            return cudaLaunchKernelEx(&cfg, gemv_w4a16_kernel<128, true>, a, p);
        }
        return cudaLaunchKernelEx(&cfg, gemv_w4a16_kernel<128, false>, a, p);
    }
    if (a.subnormal) {
        return cudaLaunchKernelEx(&cfg, gemv_w4a16_kernel<32, true>, a, p);
    }
    return cudaLaunchKernelEx(&cfg, gemv_w4a16_kernel<32, false>, a, p);
}

}  // namespace w4
