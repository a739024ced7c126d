// Decode-time W4A16 GEMV for 1..8 tokens, persistent form: the grid is two CTAs per SM (never more, never
// three on one SM) and the work -- every 256-row block of the output times every 128-channel unit of K -- is
// dealt to the CTAs as equal contiguous ranges of units ("stream-K").  A CTA therefore streams the same number
// of weight bytes whatever the shape, a range may end in the middle of one row block and continue in the next,
// and row blocks shared by several CTAs are summed by the last of them to arrive (atomic ticket, fixed
// summation order by CTA index, tickets left at zero for graph replay).
//
// Why: with a (row block, K split) grid the hardware placed 160..272 CTAs of 70..77 KB unevenly (3 on some SMs,
// none on others, clusters confined to one GPC), and the next kernel of the stream cannot pass its
// griddepcontrol.wait before the slowest CTA has left.  Here every SM slot gets one CTA of the same length.
//
// Same arithmetic as gemv.cu (mma.sync m16n8k16 with weight rows as the 16-row operand, raw nibbles as f16
// subnormals, zero point through the per-group sum of x fed in as the MMA's C operand, f32 scales applied per
// group).  Takes the place of the reference's split-K GEMV pair
// (crates/backend-gpu/src/rawcuda/assets/decode.cu:46-267, launched from
// crates/backend-gpu/src/rawcuda/w4a16_dec/kernels/decode.rs:23-127).
#include <cuda_fp16.h>

#include "gemv_common.cuh"
#include "internal.h"
#include "ptx.cuh"

namespace w4 {

namespace {

constexpr int SK_CONS_WARPS = 8;
constexpr int SK_RB_PER_WARP = CTA_RB / SK_CONS_WARPS;   // 2 row blocks per consumer warp (they share the x fragments)
constexpr int SK_THREADS = (SK_CONS_WARPS + 1) * 32;
constexpr int SK_SMEM_MAX = 113 * 1024;                   // two CTAs fit on an SM ...
constexpr int SK_SMEM_MIN = 77 * 1024;                    // ... and a third never does
constexpr int SK_MAX_STAGES = 6;
constexpr int UNIT_K = CK * TILE_K;                       // 128 input channels = one ring stage
constexpr int PART_FLOATS = GEMV_MAX_M * ROWS_PER_CTA;    // one parked partial: [8 tokens][256 rows] f32

// 32-bit arithmetic: the plan keeps units * (ctas + 1) below 2^31
__host__ __device__ __forceinline__ int sk_unit_begin(unsigned units, unsigned ctas, unsigned p) {
    return (int)(units * p / ctas);
}
// CTA that owns unit u: the largest p with sk_unit_begin(p) <= u
__host__ __device__ __forceinline__ int sk_owner(unsigned units, unsigned ctas, unsigned u) {
    return (int)(((u + 1u) * ctas - 1u) / units);
}

}  // namespace

SkPlan sk_make_plan(int k, int group, int m, int rows, int sm_count, int max_stages, int prefetch) {
    SkPlan p{};
    p.prefetch = prefetch;
    const int gpu = UNIT_K / group;   // groups per unit: 1 (g128) or 4 (g32)
    p.units_per_row = (k / TILE_K + CK - 1) / CK;
    p.rows = rows;
    p.units = (long long)rows * p.units_per_row;
    p.x_rows = m < GEMV_MAX_M ? m + 1 : m;
    const int slots = 2 * sm_count;
    int ctas = p.units < slots ? (int)p.units : slots;
    if (max_stages < 2) {
        max_stages = 2;
    }
    if (max_stages > SK_MAX_STAGES) {
        max_stages = SK_MAX_STAGES;
    }
    for (;;) {
        const int nu = (int)((p.units + ctas - 1) / ctas);
        p.nu_max = nu;
        p.x_stride = nu * UNIT_K + 32;
        int off = p.x_rows * p.x_stride * 2;
        off = (off + 127) & ~127;
        p.off_zc = off;
        off += nu * gpu * 64;
        p.off_sc = off;
        off += nu * gpu * CTA_RB * 32;
        off = (off + 1023) & ~1023;
        p.off_ring = off;
        const int room = SK_SMEM_MAX - off - (2 + 2 * SK_MAX_STAGES) * 8;
        int stages = room / STAGE_BYTES;
        if (stages >= 2 || nu == 1) {
            if (stages > max_stages) {
                stages = max_stages;
            }
            if (stages < 1) {
                stages = 1;   // a single unit per CTA with no room for two stages: k and m at their limits
            }
            p.stages = stages;
            p.off_bars = off + stages * STAGE_BYTES;
            p.total = p.off_bars + (2 + 2 * stages) * 8;
            break;
        }
        // too long a range for the staging area: more, shorter ranges (more CTAs than SM slots)
        ctas = (int)((p.units + (nu - 1) - 1) / (nu - 1));
    }
    p.ctas = ctas;
    if ((unsigned long long)p.units * (unsigned long long)(ctas + 1) >= (1ull << 31) || p.total > SK_SMEM_MAX) {
        p.ctas = 0;   // outside this kernel's index arithmetic or staging area: the caller uses gemv.cu
    }
    if (p.total < SK_SMEM_MIN) {
        p.total = SK_SMEM_MIN;
    }
    return p;
}

size_t sk_part_floats(const SkPlan& p) {
    return (size_t)p.ctas * 2 * PART_FLOATS;
}

namespace {

template <int GROUP, bool SUBN>
__global__ void __launch_bounds__(SK_THREADS, 2)
gemv_sk_kernel(const GemvArgs a, const SkPlan p) {
    constexpr int RBW = SK_RB_PER_WARP;
    constexpr int GPU_ = UNIT_K / GROUP;                                   // groups per unit
    constexpr int GROUPS_PER_KB = GROUP >= TILE_K ? 1 : TILE_K / GROUP;   // 1 for g128, 2 for g32
    extern __shared__ __align__(1024) unsigned char smem[];
    __shared__ int s_abort;
    __shared__ int s_last[2];
    __shared__ unsigned s_seq;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int C = p.units_per_row;
    const unsigned U = (unsigned)p.units;
    const int P = (int)gridDim.x, pid = (int)blockIdx.x;
    const int u0 = sk_unit_begin(U, P, pid), u1 = sk_unit_begin(U, P, pid + 1);
    const int nu = u1 - u0;
    const int nkb = a.k / TILE_K;
    const int ng = a.k / GROUP;
    const int m = a.m;
    const int S = p.stages;
    const int rg0 = u0 / C, c0 = u0 - rg0 * C;   // first unit: row block (over all segments) and unit within it

    // row block (counted over all segments) -> its segment, row block within the segment, valid 16-row blocks
    auto row_info = [&](int rg, GemvSeg& sg, int& r, int& nrbv) {
        int si = 0;
#pragma unroll
        for (int i = 1; i < GEMV_MAX_SEG; ++i) {
            if (i < a.nseg && rg >= a.seg[i].cta0) {
                si = i;
            }
        }
        sg = a.seg[si];
        r = rg - sg.cta0;
        nrbv = min(CTA_RB, sg.n / TILE_ROWS - r * CTA_RB);
    };

    const uint32_t sbase = smem_u32(smem);
    const uint32_t xbar = sbase + p.off_bars;
    auto full_bar = [&](int s) { return xbar + 8u + 8u * s; };
    auto empty_bar = [&](int s) { return xbar + 8u + 8u * (S + s); };
    volatile int* abort_flag = &s_abort;

    // optional timeline: 8 wall-clock stamps per CTA and launch (diagnostic; a.dbg is null in normal runs)
    const bool stamp = a.dbg != nullptr && pid < DBG_CTAS;
    long long* dbg = stamp ? a.dbg + ((size_t)a.dbg_seq * DBG_CTAS + pid) * DBG_STAMPS : nullptr;
    auto stamp_now = [&](int j) {
        unsigned long long ns;
        asm volatile("mov.u64 %0, %globaltimer;" : "=l"(ns));
        dbg[j] = (long long)ns;
    };

    const bool tp_on = a.tp.world > 1;
    if (threadIdx.x == 0) {
        if (stamp) {
            stamp_now(0);
            unsigned smid;
            asm volatile("mov.u32 %0, %smid;" : "=r"(smid));
            dbg[6] = smid;
            dbg[7] = nu;
        }
        s_abort = 0;
        s_last[0] = s_last[1] = 0;
        mbar_init(xbar, 1);
        mbar_init(xbar + 8u + 16u * S, 1);   // scbar
        for (int s = 0; s < S; ++s) {
            mbar_init(full_bar(s), 1);
            mbar_init(empty_bar(s), SK_CONS_WARPS);
        }
        mbar_init_fence();
    }
    float* zc_base = reinterpret_cast<float*>(smem + p.off_zc);
    if (SUBN && m < GEMV_MAX_M) {
        for (int i = threadIdx.x; i < nu * GPU_ * 16; i += blockDim.x) {
            zc_base[i] = 0.f;
        }
    }
    if (m < GEMV_MAX_M) {
        // the all-zero token row read by MMA columns >= m
        uint4* z = reinterpret_cast<uint4*>(smem + (size_t)m * p.x_stride * 2);
        for (int i = threadIdx.x; i < p.x_stride / 8; i += blockDim.x) {
            z[i] = make_uint4(0, 0, 0, 0);
        }
    }
    __syncthreads();

    // local unit j -> stage j % S: the CTA's 16 row blocks at two k-blocks (8 KB each, contiguous in T64)
    struct Cursor {
        int rg, c;        // row block and unit within it
        GemvSeg sg;
        int r, nrbv;
    };
    auto cursor_init = [&](Cursor& q) {
        q.rg = rg0;
        q.c = c0;
        row_info(q.rg, q.sg, q.r, q.nrbv);
    };
    auto cursor_next = [&](Cursor& q) {
        if (++q.c == C) {
            q.c = 0;
            ++q.rg;
            if (q.rg < p.rows) {
                row_info(q.rg, q.sg, q.r, q.nrbv);
            }
        }
    };
    auto issue_unit = [&](const Cursor& q, int s) {
        const int kbs = min(CK, nkb - q.c * CK);
        const uint32_t bytes = (uint32_t)q.nrbv * (TILE_WORDS * 4);
        const size_t nrb_seg = (size_t)(q.sg.n / TILE_ROWS);
        const unsigned char* src = reinterpret_cast<const unsigned char*>(q.sg.qt) +
                                   ((size_t)(q.c * CK) * nrb_seg + (size_t)q.r * CTA_RB) * (TILE_WORDS * 4);
        mbar_expect_tx(full_bar(s), kbs * bytes);
        for (int i = 0; i < kbs; ++i) {
            bulk_load(sbase + p.off_ring + s * STAGE_BYTES + i * KB_BYTES, src + (size_t)i * nrb_seg * (TILE_WORDS * 4),
                      bytes, full_bar(s));
        }
    };
    const bool is_producer = warp == SK_CONS_WARPS;
    const uint32_t scbar = xbar + 8u + 16u * S;
    Cursor pq;
    int pj = 0;   // next unit to issue
    if (is_producer) {
        // This CTA's scale pairs, [row block][local group][8 words]: one bulk copy per row block and run of
        // units inside a row of row blocks, requested first so that nothing queues in front of them.  Like the
        // weights they do not depend on the previous kernel of the stream.
        if (lane == 0) {
            uint32_t total = 0;
            for (int j = 0, c = c0, rg = rg0; j < nu; ++rg) {
                const int run = min(nu - j, C - c);
                GemvSeg sg;
                int r, nrbv;
                row_info(rg, sg, r, nrbv);
                total += (uint32_t)(min(run * GPU_, ng - c * GPU_) * 32 * nrbv);
                j += run;
                c = 0;
            }
            mbar_expect_tx(scbar, total);
        }
        __syncwarp();
        if (lane < CTA_RB) {
            for (int j = 0, c = c0, rg = rg0; j < nu; ++rg) {
                const int run = min(nu - j, C - c);
                GemvSeg sg;
                int r, nrbv;
                row_info(rg, sg, r, nrbv);
                if (lane < nrbv) {
                    bulk_load(sbase + p.off_sc + (uint32_t)(lane * p.nu_max + j) * (GPU_ * 32),
                              sg.st + ((size_t)(r * CTA_RB + lane) * ng + (size_t)c * GPU_) * 8,
                              (uint32_t)min(run * GPU_, ng - c * GPU_) * 32u, scbar);
                }
                j += run;
                c = 0;
            }
        }
        if (lane == 0) {
            cursor_init(pq);
            // before the previous kernel of the stream is complete only `prefetch` stages are requested: its last
            // CTAs are then summing partial results through global memory, behind whatever is queued here
            for (; pj < p.prefetch && pj < S && pj < nu; ++pj) {
                issue_unit(pq, pj);
                cursor_next(pq);
            }
        }
    }
    // Programmatic dependent launch: weights and scales do not depend on the previous kernel of the stream and
    // are already in flight while it drains; x, scratch and outputs are touched only after this wait.
    asm volatile("griddepcontrol.wait;" ::: "memory");
    if (threadIdx.x == 0) {
        // this launch's exchange number: read only now, the previous launch advances it as it ends
        s_seq = tp_on ? *reinterpret_cast<volatile unsigned*>(a.tp.seq) + 1u : 0u;
    }

    if (is_producer) {
        if (lane == 0) {
            // x of the CTA's units in local order: one copy per token and run of units inside a row block
            uint32_t total = 0;
            for (int j = 0, c = c0; j < nu;) {
                const int run = min(nu - j, C - c);
                total += (uint32_t)min(run * UNIT_K, a.k - c * UNIT_K) * 2u * (uint32_t)m;
                j += run;
                c = 0;
            }
            mbar_expect_tx(xbar, total);
            for (int j = 0, c = c0; j < nu;) {
                const int run = min(nu - j, C - c);
                const int halves = min(run * UNIT_K, a.k - c * UNIT_K);
                for (int tok = 0; tok < m; ++tok) {
                    bulk_load(sbase + (tok * p.x_stride + j * UNIT_K) * 2, a.x + (size_t)tok * a.k + (size_t)c * UNIT_K,
                              halves * 2, xbar);
                }
                j += run;
                c = 0;
            }
            if (stamp) {
                stamp_now(1);
            }
            for (; pj < S && pj < nu; ++pj) {
                issue_unit(pq, pj);
                cursor_next(pq);
            }
            int s = 0;
            uint32_t ph = 1;
            for (; pj < nu; ++pj) {
                if (!mbar_wait(empty_bar(s), ph ^ 1, abort_flag, a.status, (12 << 16) | pj)) {
                    break;
                }
                issue_unit(pq, s);
                cursor_next(pq);
                if (++s == S) {
                    s = 0;
                    ph ^= 1;
                }
            }
        }
        __syncwarp();
    } else {
        // ------------------------------------------------------------------ consumers
        bool ok = mbar_wait(xbar, 0, abort_flag, a.status, (10 << 16));
        ok = ok && mbar_wait(scbar, 0, abort_flag, a.status, (14 << 16));
        if (stamp && threadIdx.x == 0) {
            stamp_now(2);
        }
        if (SUBN && ok) {
            // zero-point term of every local group and token, -8 * sum(x), as MMA C operands: lane column t holds
            // (tokens 2t, 2t+1) x (rows g: 2^-24 per nibble unit, rows g+8: 2^-20)
            constexpr int PIECES = GROUP / 8;              // 16-byte pieces per group
            constexpr int TPP = PIECES >= 8 ? 8 : PIECES;  // threads per (group, token)
            constexpr int PER_T = PIECES / TPP;
            const int sub = threadIdx.x % TPP;
            const int ngl = nu * GPU_;
            for (int pr0 = 0; pr0 < ngl * m; pr0 += (SK_CONS_WARPS * 32) / TPP) {
                const int pr = pr0 + threadIdx.x / TPP;
                float v = 0.f;
                int grp = 0, tok = 0;
                const bool live = pr < ngl * m;
                if (live) {
                    grp = pr / m;
                    tok = pr - grp * m;
                    const uint4* xr =
                        reinterpret_cast<const uint4*>(smem + ((size_t)tok * p.x_stride + (size_t)grp * GROUP) * 2);
#pragma unroll
                    for (int j = 0; j < PER_T; ++j) {
                        const uint4 u = xr[sub * PER_T + j];
                        const float2 f0 = __half22float2(*reinterpret_cast<const __half2*>(&u.x));
                        const float2 f1 = __half22float2(*reinterpret_cast<const __half2*>(&u.y));
                        const float2 f2 = __half22float2(*reinterpret_cast<const __half2*>(&u.z));
                        const float2 f3 = __half22float2(*reinterpret_cast<const __half2*>(&u.w));
                        v += ((f0.x + f0.y) + (f1.x + f1.y)) + ((f2.x + f2.y) + (f3.x + f3.y));
                    }
                }
#pragma unroll
                for (int off = TPP / 2; off > 0; off >>= 1) {
                    v += __shfl_xor_sync(0xffffffffu, v, off);
                }
                if (live && sub == 0) {
                    float* zc = zc_base + (grp * 4 + (tok >> 1)) * 4 + (tok & 1);
                    zc[0] = -8.f * v * 5.9604644775390625e-08f;   // 2^-24
                    zc[2] = -8.f * v * 9.5367431640625e-07f;      // 2^-20
                }
            }
        }
        asm volatile("bar.sync 1, %0;" ::"n"(SK_CONS_WARPS * 32) : "memory");
        if (stamp && threadIdx.x == 0) {
            stamp_now(3);
        }

        const int rbw0 = warp * RBW;   // first row block (within the CTA's 16) of this warp
        float tot[RBW][4];
        float acc[RBW][4];
#pragma unroll
        for (int r = 0; r < RBW; ++r) {
            tot[r][0] = tot[r][1] = tot[r][2] = tot[r][3] = 0.f;
        }
        const int xrow_i = g < m ? g : m;
        const unsigned char* xp = smem + (size_t)(xrow_i * p.x_stride + 8 * t) * 2;
        const unsigned char* zp = smem + p.off_zc + t * 16;
        const unsigned char* scq = smem + p.off_sc + ((size_t)rbw0 * p.nu_max * GPU_ * 8 + g) * 4;
        const size_t sc_rb_stride = (size_t)p.nu_max * GPU_ * 32;
        const unsigned char* wbase = smem + p.off_ring + rbw0 * (TILE_WORDS * 4) + lane * 16;

        // one k-block of this warp's row blocks with everything its MMAs need, in registers
        struct KbRegs {
            uint4 w[RBW];
            uint4 x0, x1;
            float4 cz[GROUPS_PER_KB];
            uint32_t sc[RBW][GROUPS_PER_KB];
        };
        // `hk` = which k-block of the unit (0/1); zp/scq point at the unit's first group
        auto load_kb = [&](KbRegs& R, const unsigned char* wa, const unsigned char* xa, int hk) {
#pragma unroll
            for (int r = 0; r < RBW; ++r) {
                R.w[r] = *reinterpret_cast<const uint4*>(wa + r * (TILE_WORDS * 4));
            }
            R.x0 = *reinterpret_cast<const uint4*>(xa);
            R.x1 = *reinterpret_cast<const uint4*>(xa + 64);
            if (GROUP >= UNIT_K) {
                // one group per unit: its zero-point term opens k-block 0, its scale closes k-block 1
                if (hk == 0) {
                    R.cz[0] = SUBN ? *reinterpret_cast<const float4*>(zp) : make_float4(0.f, 0.f, 0.f, 0.f);
                } else {
#pragma unroll
                    for (int r = 0; r < RBW; ++r) {
                        R.sc[r][0] = *reinterpret_cast<const uint32_t*>(scq + r * sc_rb_stride);
                    }
                }
            } else {
#pragma unroll
                for (int h = 0; h < GROUPS_PER_KB; ++h) {
                    const int gi = hk * GROUPS_PER_KB + h;
                    R.cz[h] = SUBN ? *reinterpret_cast<const float4*>(zp + gi * 64) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                    for (int r = 0; r < RBW; ++r) {
                        R.sc[r][h] = *reinterpret_cast<const uint32_t*>(scq + r * sc_rb_stride + gi * 32);
                    }
                }
            }
        };
        auto expand = [&](uint32_t w, uint32_t (&fr)[4]) {
            if (SUBN) {
                nibbles_as_subnormals(w, fr);
            } else {
                dequant_word(w, fr);
            }
        };
        // half a k-block (32 k = two MMAs) of both row blocks; `init`: the chain starts from `cz`
        auto half_kblock = [&](const KbRegs& R, int hsel, bool init, const float4& cz) {
            const uint4& x = hsel ? R.x1 : R.x0;
#pragma unroll
            for (int r = 0; r < RBW; ++r) {
                uint32_t fr[4];
                expand(hsel ? R.w[r].z : R.w[r].x, fr);
                if (init) {
                    mma16816_c(acc[r], fr, x.x, x.y, cz);
                } else {
                    mma16816(acc[r], fr, x.x, x.y);
                }
                expand(hsel ? R.w[r].w : R.w[r].y, fr);
                mma16816(acc[r], fr, x.z, x.w);
            }
        };
        // end of a scale group: tot += acc * scale (nibble units; the powers of two are applied at the flush)
        auto finish_group = [&](const KbRegs& R, int h) {
#pragma unroll
            for (int r = 0; r < RBW; ++r) {
                const float2 sf = __half22float2(*reinterpret_cast<const __half2*>(&R.sc[r][h]));
                tot[r][0] = fmaf(acc[r][0], sf.x, tot[r][0]);
                tot[r][1] = fmaf(acc[r][1], sf.x, tot[r][1]);
                tot[r][2] = fmaf(acc[r][2], sf.y, tot[r][2]);
                tot[r][3] = fmaf(acc[r][3], sf.y, tot[r][3]);
            }
        };
        auto compute_kb = [&](const KbRegs& R, int hk) {
            if (GROUP >= UNIT_K) {
                half_kblock(R, 0, hk == 0, R.cz[0]);
                half_kblock(R, 1, false, R.cz[0]);
                if (hk == 1) {
                    finish_group(R, 0);
                }
            } else {
                half_kblock(R, 0, true, R.cz[0]);
                finish_group(R, 0);
                half_kblock(R, 1, true, R.cz[GROUPS_PER_KB - 1]);
                finish_group(R, GROUPS_PER_KB - 1);
            }
        };

        // the segment of the range that is being accumulated: a row block and the unit it started at
        Cursor cq;
        cursor_init(cq);
        int seg_c_begin = c0;
        bool first_seg = true;
        // end of a segment: the sums of a whole row block go to the output, those of a part of one are parked
        auto flush = [&](int c_end) {
            {
                // the powers of two of the subnormal operands, and of shifted bf16 scales (1 for f16 scales)
                const float m_lo = (SUBN ? 16777216.f : 1.f) * cq.sg.out_mul, m_hi = (SUBN ? 1048576.f : 1.f) * cq.sg.out_mul;
#pragma unroll
                for (int r = 0; r < RBW; ++r) {
                    tot[r][0] *= m_lo;
                    tot[r][1] *= m_lo;
                    tot[r][2] *= m_hi;
                    tot[r][3] *= m_hi;
                }
            }
            const bool whole = seg_c_begin == 0 && c_end == C;
            float* park = a.part + ((size_t)pid * 2 + (first_seg ? 0 : 1)) * PART_FLOATS;
#pragma unroll
            for (int r = 0; r < RBW; ++r) {
                if (rbw0 + r < cq.nrbv) {
                    const int lr0 = (rbw0 + r) * TILE_ROWS + g, lr1 = lr0 + 8;
                    const int row0 = cq.r * ROWS_PER_CTA + lr0, row1 = row0 + 8;
#pragma unroll
                    for (int j = 0; j < 2; ++j) {
                        const int tok = 2 * t + j;
                        if (tok < m) {
                            if (!whole) {
                                park[tok * ROWS_PER_CTA + lr0] = tot[r][j];
                                park[tok * ROWS_PER_CTA + lr1] = tot[r][2 + j];
                            } else if (tp_on) {
                                float* o = tp_own_area(a.tp, s_seq);
                                o[(size_t)tok * a.tp.max_rows + row0] = tot[r][j];
                                o[(size_t)tok * a.tp.max_rows + row1] = tot[r][2 + j];
                            } else if (a.out_f16) {
                                __half* o = reinterpret_cast<__half*>(cq.sg.out) + (size_t)tok * cq.sg.n;
                                o[row0] = __float2half_rn(tot[r][j]);
                                o[row1] = __float2half_rn(tot[r][2 + j]);
                            } else {
                                float* o = reinterpret_cast<float*>(cq.sg.out) + (size_t)tok * cq.sg.n;
                                o[row0] = tot[r][j];
                                o[row1] = tot[r][2 + j];
                            }
                        }
                    }
                }
                tot[r][0] = tot[r][1] = tot[r][2] = tot[r][3] = 0.f;
            }
            first_seg = false;
            seg_c_begin = 0;
        };

        // Software pipeline over k-blocks: the registers of the next k-block are loaded before the MMAs of the
        // current one, and a stage goes back to the producer as soon as both of its k-blocks are in registers.
        static_assert(CK == 2, "the pipeline below is written for two k-blocks per stage");
        int s = 0;
        uint32_t ph = 0;
        KbRegs A, B;
        ok = ok && mbar_wait(full_bar(0), 0, abort_flag, a.status, (11 << 16));
        if (ok) {
            load_kb(A, wbase, xp, 0);
            for (int j = 0; j < nu; ++j) {
                const bool has_b = cq.c * CK + 1 < nkb;   // false only for a ragged last unit of a row (g32)
                if (has_b) {
                    load_kb(B, wbase + s * STAGE_BYTES + KB_BYTES, xp + 128, 1);
                }
                compute_kb(A, 0);
                __syncwarp();
                if (lane == 0) {
                    mbar_arrive(empty_bar(s));
                }
                if (++s == S) {
                    s = 0;
                    ph ^= 1;
                }
                xp += UNIT_K * 2;
                zp += GPU_ * 64;
                scq += GPU_ * 32;
                if (j + 1 < nu) {
                    ok = mbar_wait(full_bar(s), ph, abort_flag, a.status, (11 << 16) | (j + 1));
                    if (!ok) {
                        break;
                    }
                    load_kb(A, wbase + s * STAGE_BYTES, xp, 0);
                }
                if (has_b) {
                    compute_kb(B, 1);
                }
                const int c_end = cq.c + 1;
                if (c_end == C || j + 1 == nu) {
                    flush(c_end);
                }
                cursor_next(cq);
            }
        }
    }
    if (stamp && threadIdx.x == 0) {
        stamp_now(4);
    }
    // the next kernel of the stream may start its weight stream now (it waits for our completion before
    // touching x, scratch or outputs)
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    // ---- row blocks shared with other CTAs: the last contributor to arrive sums the parked partials -------
    // slot 0: the range's first row block, slot 1: its last one (when different); whole row blocks never park.
    // (Polling the parked words instead of taking tickets was tried: loads that are coherent across the two
    // dies' L2 cost as much as the fence and the ticket together, and cache-global loads were seen to miss
    // another CTA's store until the wait's limit.)
    const int rg_last = (u1 - 1) / C;
    int prow[2];
    prow[0] = (c0 == 0 && u1 >= (rg0 + 1) * C) ? -1 : rg0;
    prow[1] = (rg_last != rg0 && u1 != (rg_last + 1) * C) ? rg_last : -1;
    __threadfence();
    __syncthreads();
    if (stamp && threadIdx.x == 0) {
        stamp_now(8);   // partial sums visible
    }
    if (threadIdx.x == 0 && !*abort_flag) {
        for (int sl = 0; sl < 2; ++sl) {
            if (prow[sl] >= 0) {
                const unsigned ub = (unsigned)(prow[sl] * C);
                const int ncontrib = sk_owner(U, P, ub + C - 1) - sk_owner(U, P, ub) + 1;
                const unsigned ticket = atomicAdd(a.counters + prow[sl], 1u);
                s_last[sl] = ticket == (unsigned)ncontrib - 1u;
            }
        }
        __threadfence();   // the parked sums of the earlier contributors, ordered after the tickets
    }
    __syncthreads();
    if (stamp && threadIdx.x == 0) {
        stamp_now(9);   // tickets taken
        dbg[10] = s_last[0] + 2 * s_last[1];
    }
    for (int sl = 0; sl < 2; ++sl) {
        if (prow[sl] < 0 || !s_last[sl]) {
            continue;
        }
        const int rg = prow[sl];
        const unsigned ub = (unsigned)(rg * C);
        const int p_first = sk_owner(U, P, ub), p_last = sk_owner(U, P, ub + C - 1);
        // only the first contributor can hold this row block as a later segment of its range (slot 1)
        const int slot_first = sk_unit_begin(U, P, p_first) / C == rg ? 0 : 1;
        GemvSeg sg;
        int r, nrbv;
        row_info(rg, sg, r, nrbv);
        // four rows per thread; all contributors' loads of a batch are in flight before the first add
        const int nq = nrbv * (TILE_ROWS / 4);
        constexpr int BATCH = 16;
        for (int i = threadIdx.x; i < nq * m; i += blockDim.x) {
            const int tok = i / nq, l4 = i - tok * nq;
            const float4* src = reinterpret_cast<const float4*>(a.part + tok * ROWS_PER_CTA) + l4;
            float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
            for (int pb = p_first; pb <= p_last; pb += BATCH) {
                float4 v[BATCH];
#pragma unroll
                for (int q = 0; q < BATCH; ++q) {
                    const int pp = min(pb + q, p_last);
                    const size_t slot = (size_t)pp * 2 + (pp == p_first ? slot_first : 0);
                    v[q] = __ldcg(src + slot * (PART_FLOATS / 4));
                }
#pragma unroll
                for (int q = 0; q < BATCH; ++q) {
                    if (pb + q <= p_last) {
                        sum.x += v[q].x;
                        sum.y += v[q].y;
                        sum.z += v[q].z;
                        sum.w += v[q].w;
                    }
                }
            }
            const int row = r * ROWS_PER_CTA + l4 * 4;
            if (tp_on) {
                *reinterpret_cast<float4*>(tp_own_area(a.tp, s_seq) + (size_t)tok * a.tp.max_rows + row) = sum;
            } else if (a.out_f16) {
                const __half2 h0 = __floats2half2_rn(sum.x, sum.y), h1 = __floats2half2_rn(sum.z, sum.w);
                uint2 pk;
                pk.x = *reinterpret_cast<const uint32_t*>(&h0);
                pk.y = *reinterpret_cast<const uint32_t*>(&h1);
                *reinterpret_cast<uint2*>(reinterpret_cast<__half*>(sg.out) + (size_t)tok * sg.n + row) = pk;
            } else {
                *reinterpret_cast<float4*>(reinterpret_cast<float*>(sg.out) + (size_t)tok * sg.n + row) = sum;
            }
        }
        if (threadIdx.x == 0) {
            a.counters[rg] = 0;   // ready for the next launch (graph replay needs no memset)
        }
    }
    if (tp_on) {
        // every row block this CTA finished (whole ones of its range, and shared ones it reduced) is exchanged
        const int rf0 = (u0 + C - 1) / C, rf1 = u1 / C;
        for (int rg = rf0; rg < rf1; ++rg) {
            GemvSeg sg;
            int r, nrbv;
            row_info(rg, sg, r, nrbv);
            tp_exchange(a, sg, r * CTA_RB, nrbv * TILE_ROWS, &s_seq, abort_flag, (unsigned)p.rows, dbg);
        }
        for (int sl = 0; sl < 2; ++sl) {
            if (prow[sl] >= 0 && s_last[sl]) {
                GemvSeg sg;
                int r, nrbv;
                row_info(prow[sl], sg, r, nrbv);
                tp_exchange(a, sg, r * CTA_RB, nrbv * TILE_ROWS, &s_seq, abort_flag, (unsigned)p.rows, dbg);
            }
        }
    }
    if (stamp && threadIdx.x == 0) {
        stamp_now(5);
    }
}

}  // namespace

cudaError_t gemv_sk_init_device() {
    cudaError_t e;
#define W4_SET(K) \
    e = cudaFuncSetAttribute(K, cudaFuncAttributeMaxDynamicSharedMemorySize, SK_SMEM_MAX); \
    if (e != cudaSuccess) return e;
    W4_SET((gemv_sk_kernel<128, true>))
    W4_SET((gemv_sk_kernel<128, false>))
    W4_SET((gemv_sk_kernel<32, true>))
    W4_SET((gemv_sk_kernel<32, false>))
#undef W4_SET
    return cudaSuccess;
}

cudaError_t launch_gemv_sk(const GemvArgs& a, const SkPlan& p, cudaStream_t st) {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(p.ctas);
    cfg.blockDim = dim3(SK_THREADS);
    cfg.dynamicSmemBytes = p.total;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    int na = 0;
    if (a.pdl) {
        attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[na].val.programmaticStreamSerializationAllowed = 1;
        ++na;
    }
    cfg.attrs = attr;
    cfg.numAttrs = na;
    if (a.group == 128) {
        return a.subnormal ? cudaLaunchKernelEx(&cfg, gemv_sk_kernel<128, true>, a, p)
                           : cudaLaunchKernelEx(&cfg, gemv_sk_kernel<128, false>, a, p);
    }
    return a.subnormal ? cudaLaunchKernelEx(&cfg, gemv_sk_kernel<32, true>, a, p)
                       : cudaLaunchKernelEx(&cfg, gemv_sk_kernel<32, false>, a, p);
}

}  // namespace w4
