// Decode-time W4A16 split-K GEMV for 1..8 tokens:  y[m][n] = sum_k x[m][k] * (q[n][k]-8) * s[n][k/group],
// (row block, K split) form: grid (256-row blocks, K splits).  Dec::gemv uses it for 5..8 tokens, the MoE decode
// path uses its table-driven "grouped" mode; up to 4 tokens run the persistent form in gemv_sk.cu.
//
// Takes the place of the reference's split-K GEMV pair (crates/backend-gpu/src/rawcuda/assets/decode.cu:46-267,
// launched from crates/backend-gpu/src/rawcuda/w4a16_dec/kernels/decode.rs:23-127) and of its FFMA
// small-batch family (crates/backend-gpu/src/rawcuda/assets/gptq4.cu:44-723).  Differences by design:
//   * the 16 rows of each mma.sync m16n8k16 are WEIGHT rows and the 8 columns are tokens, so
//     m = 1..8 all use the same kernel and no MMA row is padding;
//   * weights never become rounded f16 values: the MMA multiplies the raw nibble (as an exact f16
//     subnormal, nibble * 2^-24 or 2^-20) by x; the zero point 8 enters as the C operand of a group's first
//     MMA (-8 * sum of x over the group, pre-scaled), the f32 group scale is applied to the accumulator once
//     per group and the power of two once at the end;
//   * a CTA owns 256 weight rows and a K range.  One producer lane streams them through a ring of
//     16 KB stages in shared memory with 8 KB bulk (TMA) copies -- the 16 row blocks of a CTA are
//     contiguous at each k-block in the T64 layout -- and 8 consumer warps (two row blocks each, sharing
//     the x fragments) keep the next k-block in registers while they multiply the current one, wait only on a
//     "full" mbarrier and arrive on an "empty" one as soon as a stage is in registers;
//   * the K splits of a row block form a thread-block cluster and sum their partials through distributed
//     shared memory (2..8 splits); otherwise the partials go to global scratch and the last CTA to arrive
//     reduces them (atomic ticket, no spin).  Either way: fixed summation order, no second launch, and the
//     tickets are left at zero for graph replay;
//   * launched with programmatic stream serialization: the weight stream starts while the previous
//     kernel of the stream drains; x, scratch and outputs are touched only after griddepcontrol.wait.
// The kernel is HBM-bound.
#include <cuda_fp16.h>

#include "gemv_common.cuh"
#include "internal.h"
#include "ptx.cuh"

namespace w4 {

namespace {

constexpr int MAX_STAGES = 8;

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

constexpr int GEMV_SMEM_LIMIT = 112 * 1024;       // two CTAs per SM
constexpr int SC_STAGE_MAX = 32 * 1024;           // most scale bytes a CTA stages in shared memory

struct SmemPlan {
    int x_stride;   // halves per token row (byte stride = 64 mod 128: conflict-free 128-bit reads)
    int x_rows;     // token rows staged (m, plus one all-zero row when m < 8)
    int off_xsum;   // f32 [groups][4 lane columns][4]: the zero-point term of each group as MMA C operands
    int off_sc;     // u32 [16 row blocks][groups][8]: this CTA's scale pairs (when sc_staged)
    int sc_staged;  // 1: the scales of the CTA's rows and K range are copied to shared memory up front
    int off_ring;   // stages x STAGE_BYTES, 1024-byte aligned
    int off_bars;   // xbar, full[stages], empty[stages], scbar
    int stages;
    int total;
};

__host__ SmemPlan make_plan(int k, int group, int m, int ksplit, int stages) {
    SmemPlan p;
    p.stages = stages < 2 ? 2 : (stages > MAX_STAGES ? MAX_STAGES : stages);
    const int halves = max_split_kblocks(k, group, ksplit) * TILE_K;
    const int ngl = halves / group;
    p.x_stride = halves + 32;
    p.x_rows = m < GEMV_MAX_M ? m + 1 : m;
    int off = p.x_rows * p.x_stride * 2;
    off = (off + 127) & ~127;
    p.off_xsum = off;
    off += ngl * 16 * 4;
    p.off_sc = off;
    const int sc_bytes = ngl * CTA_RB * 32;
    const int rest = 1024 + p.stages * STAGE_BYTES + (2 + 2 * p.stages) * 8;
    p.sc_staged = sc_bytes <= SC_STAGE_MAX && off + sc_bytes + rest <= GEMV_SMEM_LIMIT;
    if (p.sc_staged) {
        off += sc_bytes;
    }
    off = (off + 1023) & ~1023;
    p.off_ring = off;
    off += p.stages * STAGE_BYTES;
    p.off_bars = off;
    off += (2 + 2 * p.stages) * 8;
    p.total = off;
    return p;
}

// CONS_WARPS consumer warps (8 or 16) own 16/CONS_WARPS row blocks each; warp CONS_WARPS is the producer.
template <int GROUP, bool SUBN, int CONS_WARPS>
__global__ void __launch_bounds__((CONS_WARPS + 1) * 32)
gemv_w4a16_kernel(const GemvArgs a, const SmemPlan p) {
    constexpr int RB_PER_WARP = CTA_RB / CONS_WARPS;
    extern __shared__ __align__(1024) unsigned char smem[];
    __shared__ int s_is_last;
    __shared__ int s_abort;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int split = blockIdx.y;
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
    GemvSeg sg = a.seg[si];
    int m_loc = a.m;                                       // tokens of this CTA (grouped mode: rows of its tile)
    const uint16_t* x_loc = a.x;
    int rb_cta0 = ((int)blockIdx.x - sg.cta0) * CTA_RB;    // first row block of this CTA within its output
    int rb_w0 = rb_cta0;                                   // ... and within the resident weight matrix
    int row_base = 0;                                      // sorted row of token 0 (grouped mode)
    if (a.grouped) {
        if (a.tables_fresh) {
            asm volatile("griddepcontrol.wait;" ::: "memory");
        }
        const int ti = (int)blockIdx.x / a.ctas_per_seg;
        if (ti >= *a.num_tiles) {
            return;  // the grid is sized for the worst case; whole clusters leave together
        }
        row_base = a.tile_row0[ti];
        m_loc = a.tile_rows[ti];
        x_loc = x_loc + (size_t)row_base * a.k;
        rb_cta0 = ((int)blockIdx.x % a.ctas_per_seg) * CTA_RB;
        rb_w0 = (a.tile_expert[ti] - a.expert0) * (sg.n / TILE_ROWS) + rb_cta0;
        sg.out = a.out_f16 ? (void*)(reinterpret_cast<__half*>(sg.out) + (size_t)row_base * sg.n)
                           : (void*)(reinterpret_cast<float*>(sg.out) + (size_t)row_base * sg.n);
    }
    const int nrb_seg = sg.n / TILE_ROWS;
    const int nrb_pitch = a.nrb_w > 0 ? a.nrb_w : nrb_seg;
    const int nrbv = min(CTA_RB, nrb_seg - rb_cta0);             // valid row blocks in this CTA

    int kb0, kb1;
    split_range(a.k, GROUP, a.ksplit, split, &kb0, &kb1);
    const int nloc = kb1 - kb0;                      // k-blocks of this split
    const int halves = nloc * TILE_K;
    const int ngl = halves / GROUP;                  // scale groups of this split
    const int nchunks = (nloc + CK - 1) / CK;
    const int S = p.stages;

    const uint32_t sbase = smem_u32(smem);
    const uint32_t xbar = sbase + p.off_bars;
    auto full_bar = [&](int s) { return xbar + 8u + 8u * s; };
    auto empty_bar = [&](int s) { return xbar + 8u + 8u * (S + s); };
    const uint32_t scbar = xbar + 8u + 16u * S;
    volatile int* abort_flag = &s_abort;
    // optional timeline: 8 wall-clock stamps per CTA and launch (diagnostic; a.dbg is null in normal runs)
    const int dbg_cta = (int)(blockIdx.y * gridDim.x + blockIdx.x);
    const bool stamp = a.dbg != nullptr && dbg_cta < DBG_CTAS;
    long long* dbg = stamp ? a.dbg + ((size_t)a.dbg_seq * DBG_CTAS + dbg_cta) * DBG_STAMPS : nullptr;
    auto stamp_now = [&](int j) {
        unsigned long long ns;
        asm volatile("mov.u64 %0, %globaltimer;" : "=l"(ns));
        dbg[j] = (long long)ns;
    };

    __shared__ unsigned s_seq;
    const bool tp_on = a.tp.world > 1;
    if (threadIdx.x == 0) {
        if (stamp) {
            stamp_now(0);   // CTA entry
            unsigned smid;
            asm volatile("mov.u32 %0, %smid;" : "=r"(smid));
            dbg[6] = smid;
            dbg[7] = nchunks;
        }
        s_abort = 0;
        mbar_init(xbar, 1);
        mbar_init(scbar, 1);
        for (int s = 0; s < S; ++s) {
            mbar_init(full_bar(s), 1);
            mbar_init(empty_bar(s), CONS_WARPS);
        }
        mbar_init_fence();
    }
    if (SUBN && m_loc < GEMV_MAX_M) {
        float* xsum = reinterpret_cast<float*>(smem + p.off_xsum);
        for (int i = threadIdx.x; i < ngl * 16; i += blockDim.x) {
            xsum[i] = 0.f;
        }
    }
    // the all-zero token row read by MMA columns >= m
    if (m_loc < GEMV_MAX_M) {
        uint4* z = reinterpret_cast<uint4*>(smem + (size_t)m_loc * p.x_stride * 2);
        for (int i = threadIdx.x; i < p.x_stride / 8; i += blockDim.x) {
            z[i] = make_uint4(0, 0, 0, 0);
        }
    }
    __syncthreads();

    // chunk c -> stage c % S: CK bulk copies of the CTA's rows at one k-block each (contiguous in T64)
    const unsigned char* wsrc = reinterpret_cast<const unsigned char*>(sg.qt) +
                                ((size_t)kb0 * nrb_pitch + rb_w0) * (TILE_WORDS * 4);
    const size_t kb_pitch = (size_t)nrb_pitch * (TILE_WORDS * 4);
    auto issue_chunk = [&](int c, int s) {
        const int kbs = min(CK, nloc - c * CK);
        const uint32_t bytes = (uint32_t)nrbv * (TILE_WORDS * 4);
        mbar_expect_tx(full_bar(s), kbs * bytes);
        for (int i = 0; i < kbs; ++i) {
            bulk_load(sbase + p.off_ring + s * STAGE_BYTES + i * KB_BYTES, wsrc + (size_t)(c * CK + i) * kb_pitch, bytes,
                      full_bar(s));
        }
    };
    const bool is_producer = warp == CONS_WARPS;
    if (is_producer) {
        if (p.sc_staged) {
            // this CTA's scale pairs, [row block][group][8]: one bulk copy per row block (contiguous along K), requested
            // first so that nothing queues in front of them; like the weights they do not depend on the previous kernel
            const int ng_all = a.k / GROUP;
            const size_t grp_first = (size_t)kb0 * GROUPS_PER_KB / KB_PER_GROUP;
            if (lane == 0) {
                mbar_expect_tx(scbar, (uint32_t)(nrbv * ngl * 32));
            }
            __syncwarp();
            if (lane < nrbv) {
                bulk_load(sbase + p.off_sc + (uint32_t)(lane * ngl * 32), sg.st + ((size_t)(rb_w0 + lane) * ng_all + grp_first) * 8,
                          (uint32_t)(ngl * 32), scbar);
            }
        }
        if (lane == 0) {
            for (int c = 0; c < S && c < nchunks; ++c) {
                issue_chunk(c, c);
            }
        }
    }
    // Programmatic dependent launch: the weight copies above do not depend on the previous kernel in the
    // stream, so they are already in flight while it drains.  Everything below reads x or writes
    // scratch/outputs and must wait for it.  (griddepcontrol does nothing in an ordinary launch.)
    if (a.pdl == 2) {
        // early trigger: the next kernel's CTAs take whatever SM slots this grid leaves free and prefetch
        // their first weight stages while this kernel computes (they still wait for it before using x)
        asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    }
    asm volatile("griddepcontrol.wait;" ::: "memory");
    if (threadIdx.x == 0) {
        // this launch's exchange number: read only now, the previous launch advances it as it ends
        s_seq = tp_on ? *reinterpret_cast<volatile unsigned*>(a.tp.seq) + 1u : 0u;
        mbar_expect_tx(xbar, m_loc * halves * 2);
    }
    if (warp == 0) {
        // one lane per token: the row lookups of a grouped call are independent loads, not a chain
        __syncwarp();
        if (lane < m_loc) {
            const uint16_t* xr = x_loc + (size_t)lane * a.k;
            if (a.x_slot_of_pos != nullptr) {
                // the activations were not gathered into sorted order: fetch the token's row
                xr = a.x + (size_t)(a.x_slot_of_pos[row_base + lane] / a.x_slots_per_token) * a.k;
            }
            bulk_load(sbase + lane * p.x_stride * 2, xr + (size_t)kb0 * TILE_K, halves * 2, xbar);
        }
        if (stamp && lane == 0) {
            stamp_now(1);   // the previous kernel of the stream is complete; x requested
        }
    }

    if (is_producer) {
        // ------------------------------------------------------------------ producer: refill freed stages
        if (lane == 0) {
            int s = 0;
            uint32_t ph = 1;   // chunk c >= S reuses stage s after the consumers' (c / S)-th release of it
            for (int c = S; c < nchunks; ++c) {
                if (!mbar_wait(empty_bar(s), ph ^ 1, abort_flag, a.status, (12 << 16) | c)) {
                    break;
                }
                issue_chunk(c, s);
                if (++s == S) {
                    s = 0;
                    ph ^= 1;
                }
            }
        }
        __syncwarp();
    }
    bool ok = true;
    if (!is_producer) {
        ok = mbar_wait(xbar, 0, abort_flag, a.status, (10 << 16));
        if (ok && p.sc_staged) {
            ok = mbar_wait(scbar, 0, abort_flag, a.status, (14 << 16));
        }
        if (stamp && threadIdx.x == 0) {
            stamp_now(2);   // x and scales in shared memory
        }
        if (SUBN && ok) {
            // xsum[grp][tok] = -8 * sum_{k in grp} x[tok][k] for tok < m (entries of tokens >= m stay zero):
            // a few threads per (group, token), partial sums combined with shuffles.
            float* xsum = reinterpret_cast<float*>(smem + p.off_xsum);
            constexpr int PIECES = GROUP / 8;              // 16-byte pieces per group
            constexpr int TPP = PIECES >= 8 ? 8 : PIECES;  // threads per (group, token): 8 (g128) or 4 (g32)
            constexpr int PER_T = PIECES / TPP;
            const int sub = threadIdx.x % TPP;
            for (int pr0 = 0; pr0 < ngl * m_loc; pr0 += (CONS_WARPS * 32) / TPP) {
                const int pr = pr0 + threadIdx.x / TPP;
                float v = 0.f;
                int grp = 0, tok = 0;
                const bool live = pr < ngl * m_loc;
                if (live) {
                    grp = pr / m_loc;
                    tok = pr - grp * m_loc;
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
                    // C operands of the group's first MMA: rows g carry 2^-24 per nibble unit, rows g+8 2^-20
                    float* zc = xsum + (grp * 4 + (tok >> 1)) * 4 + (tok & 1);
                    zc[0] = -8.f * v * 5.9604644775390625e-08f;
                    zc[2] = -8.f * v * 9.5367431640625e-07f;
                }
            }
        }
        // consumers only: the producer warp is busy refilling the ring
        asm volatile("bar.sync 1, %0;" ::"n"(CONS_WARPS * 32) : "memory");
        if (stamp && threadIdx.x == 0) {
            stamp_now(3);   // main loop starts
        }
    }
    // ---------------------------------------------------------------------- consumers: stream and accumulate
    float tot[RB_PER_WARP][4];
#pragma unroll
    for (int r = 0; r < RB_PER_WARP; ++r) {
        tot[r][0] = tot[r][1] = tot[r][2] = tot[r][3] = 0.f;
    }
    const int rbw0 = warp * RB_PER_WARP;  // first row block (within the CTA) of this warp
    const bool warp_active = !is_producer && rbw0 < nrbv;
    const int nvalid = warp_active ? min(RB_PER_WARP, nrbv - rbw0) : 0;
    if (warp_active && ok) {
        // scale pairs of rows (g, g+8), one 32-bit word per group at a stride of 8 words: from the staged copy
        // in shared memory, else straight from global memory
        const uint32_t* scp[RB_PER_WARP];
#pragma unroll
        for (int r = 0; r < RB_PER_WARP; ++r) {
            const int rr = r < nvalid ? r : 0;
            if (p.sc_staged) {
                scp[r] = reinterpret_cast<const uint32_t*>(smem + p.off_sc) + (size_t)(rbw0 + rr) * ngl * 8 + g;
            } else {
                const int ng = a.k / GROUP;
                const size_t grp0 = (size_t)kb0 * GROUPS_PER_KB / KB_PER_GROUP;
                scp[r] = sg.st + ((size_t)(rb_w0 + rbw0 + rr) * ng + grp0) * 8 + g;
            }
        }
        // B fragment source: token g (the zero row when g >= m), this lane's 8 k of each half k-block
        const int xrow_i = g < m_loc ? g : m_loc;
        const unsigned char* xp = smem + (size_t)(xrow_i * p.x_stride + 8 * t) * 2;
        const unsigned char* zp = smem + p.off_xsum + t * 16;
        const unsigned char* wbase = smem + p.off_ring + rbw0 * (TILE_WORDS * 4) + lane * 16;

        float acc[RB_PER_WARP][4];
        uint32_t sc[RB_PER_WARP];
#pragma unroll
        for (int r = 0; r < RB_PER_WARP; ++r) {
            sc[r] = *scp[r];
        }
        int gl = 0;

        // one k-block of this warp's row blocks and the matching x fragments, in registers
        struct KbRegs {
            uint4 w[RB_PER_WARP];
            uint4 x0, x1;
        };
        auto load_kb = [&](KbRegs& R, const unsigned char* wa, const unsigned char* xa) {
#pragma unroll
            for (int r = 0; r < RB_PER_WARP; ++r) {
                R.w[r] = *reinterpret_cast<const uint4*>(wa + r * (TILE_WORDS * 4));
            }
            R.x0 = *reinterpret_cast<const uint4*>(xa);
            R.x1 = *reinterpret_cast<const uint4*>(xa + 64);
        };
        auto expand = [&](uint32_t w, uint32_t (&fr)[4]) {
            if (SUBN) {
                nibbles_as_subnormals(w, fr);
            } else {
                dequant_word(w, fr);
            }
        };
        // end of a scale group: tot += acc * scale (still in nibble units: the powers of two come at the end)
        auto finish_group = [&]() {
            ++gl;
#pragma unroll
            for (int r = 0; r < RB_PER_WARP; ++r) {
                const float2 sf = __half22float2(*reinterpret_cast<const __half2*>(&sc[r]));
                if (gl < ngl) {
                    sc[r] = scp[r][gl * 8];  // the next group's scales
                }
                tot[r][0] = fmaf(acc[r][0], sf.x, tot[r][0]);
                tot[r][1] = fmaf(acc[r][1], sf.x, tot[r][1]);
                tot[r][2] = fmaf(acc[r][2], sf.y, tot[r][2]);
                tot[r][3] = fmaf(acc[r][3], sf.y, tot[r][3]);
            }
        };
        // half a k-block (32 k = two MMAs) of every row block; `init` opens a scale group: the chain starts from
        // the group's zero-point term, -8 * sum(x), pre-scaled to the nibble units of the accumulator
        auto half_kblock = [&](const KbRegs& R, int hsel, bool init) {
            const uint4& x = hsel ? R.x1 : R.x0;
            float4 cz = make_float4(0.f, 0.f, 0.f, 0.f);
            if (init && SUBN) {
                cz = *reinterpret_cast<const float4*>(zp);
                zp += 64;
            }
#pragma unroll
            for (int r = 0; r < RB_PER_WARP; ++r) {
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
        // one k-block; `first`/`last`: it opens / closes a scale group (g128); g32 groups are half k-blocks
        auto compute_kb = [&](const KbRegs& R, bool first, bool last) {
            half_kblock(R, 0, first || GROUP < TILE_K);
            if (GROUP < TILE_K) {
                finish_group();
            }
            half_kblock(R, 1, GROUP < TILE_K);
            if (GROUP < TILE_K || last) {
                finish_group();
            }
        };

        // Software pipeline over k-blocks: the registers of the next k-block are loaded before the MMAs of the
        // current one, and a stage goes back to the producer as soon as both of its k-blocks are in registers.
        // Splits are whole groups, so a g128 chunk (two k-blocks) is exactly one group.
        static_assert(CK == 2, "the pipeline below is written for two k-blocks per stage");
        int s = 0;
        uint32_t ph = 0;
        KbRegs A, B;
        ok = mbar_wait(full_bar(0), 0, abort_flag, a.status, (11 << 16));
        if (ok) {
            load_kb(A, wbase, xp);
            for (int c = 0; c < nchunks; ++c) {
                const bool has_b = c * CK + 1 < nloc;   // false only for a ragged last chunk (g32)
                if (has_b) {
                    load_kb(B, wbase + s * STAGE_BYTES + KB_BYTES, xp + 128);
                }
                compute_kb(A, true, false);
                __syncwarp();
                if (lane == 0) {
                    mbar_arrive(empty_bar(s));
                }
                if (++s == S) {
                    s = 0;
                    ph ^= 1;
                }
                xp += CK * 128;
                if (c + 1 < nchunks) {
                    ok = mbar_wait(full_bar(s), ph, abort_flag, a.status, (11 << 16) | (c + 1));
                    if (!ok) {
                        break;
                    }
                    load_kb(A, wbase + s * STAGE_BYTES, xp);
                }
                if (has_b) {
                    compute_kb(B, false, true);
                }
            }
        }
        {
            // the powers of two of the subnormal operands, and of shifted bf16 scales (1 for f16 scales)
            const float m_lo = (SUBN ? 16777216.f : 1.f) * sg.out_mul, m_hi = (SUBN ? 1048576.f : 1.f) * sg.out_mul;
#pragma unroll
            for (int r = 0; r < RB_PER_WARP; ++r) {
                tot[r][0] *= m_lo;
                tot[r][1] *= m_lo;
                tot[r][2] *= m_hi;
                tot[r][3] *= m_hi;
            }
        }
    } else if (!is_producer && ok) {
        // a consumer warp without rows still releases every stage
        int s = 0;
        uint32_t ph = 0;
        for (int c = 0; c < nchunks; ++c) {
            if (!mbar_wait(full_bar(s), ph, abort_flag, a.status, (13 << 16) | c)) {
                break;
            }
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(empty_bar(s));
            }
            if (++s == S) {
                s = 0;
                ph ^= 1;
            }
        }
    }
    if (stamp && threadIdx.x == 0) {
        stamp_now(4);   // main loop done (warp 0)
    }

    // the next kernel of the stream may start its weight stream now (it waits for our completion
    // before touching x, scratch or outputs)
    if (a.pdl != 2) {
        asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    }

    // tot[r][0],[1]: row g, tokens 2t, 2t+1 ; tot[r][2],[3]: row g+8, tokens 2t, 2t+1
    if (a.ksplit == 1 && a.glu) {
        // interleaved gate / up row blocks: this warp's two row blocks are the gate and the up rows of the same 16
        // outputs, so the activation is applied here and [rows][n/2] f16 is stored
        if (RB_PER_WARP == 2 && nvalid == 2) {
            const int orow0 = ((rb_cta0 + rbw0) / 2) * TILE_ROWS + g, orow1 = orow0 + 8;
            const int nh = sg.n / 2;
            __half* ob = reinterpret_cast<__half*>(a.seg[0].out) + (size_t)row_base * nh;
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                const int tok = 2 * t + j;
                if (tok < m_loc) {
                    ob[(size_t)tok * nh + orow0] = silu_mul_f16(tot[0][j], tot[RB_PER_WARP - 1][j]);
                    ob[(size_t)tok * nh + orow1] = silu_mul_f16(tot[0][2 + j], tot[RB_PER_WARP - 1][2 + j]);
                }
            }
        }
        if (stamp && threadIdx.x == 0) {
            stamp_now(5);
        }
        return;
    }
    if (a.ksplit == 1) {
#pragma unroll
        for (int r = 0; r < RB_PER_WARP; ++r) {
            if (r < nvalid) {
                const int row0 = (rb_cta0 + rbw0 + r) * TILE_ROWS + g, row1 = row0 + 8;
#pragma unroll
                for (int j = 0; j < 2; ++j) {
                    const int tok = 2 * t + j;
                    if (tok < m_loc) {
                        if (a.row_w != nullptr) {
                            const float rw = a.row_w[row_base + tok];
                            tot[r][j] = mul_row_w(tot[r][j], rw);
                            tot[r][2 + j] = mul_row_w(tot[r][2 + j], rw);
                        }
                        if (tp_on) {
                            float* o = tp_own_area(a.tp, s_seq);
                            o[(size_t)tok * a.tp.max_rows + row0] = tot[r][j];
                            o[(size_t)tok * a.tp.max_rows + row1] = tot[r][2 + j];
                        } else if (a.out_f16) {
                            __half* o = reinterpret_cast<__half*>(sg.out) + (size_t)tok * sg.n;
                            o[row0] = __float2half_rn(tot[r][j]);
                            o[row1] = __float2half_rn(tot[r][2 + j]);
                        } else {
                            float* o = reinterpret_cast<float*>(sg.out) + (size_t)tok * sg.n;
                            o[row0] = tot[r][j];
                            o[row1] = tot[r][2 + j];
                        }
                    }
                }
            }
        }
        if (tp_on) {
            tp_exchange(a, sg, rb_cta0, nrbv * TILE_ROWS, &s_seq, abort_flag, gridDim.x);
        }
        if (stamp && threadIdx.x == 0) {
            stamp_now(5);
        }
        return;
    }

    if (a.cluster) {
        // split-K inside a thread-block cluster: the ksplit CTAs of this row block park their partial sums in
        // their own shared memory and every CTA sums a slice of the rows over all splits, in split order,
        // through distributed shared memory -- no global round trip, no ticket.
        __syncthreads();  // the weight ring is idle now; its first stage becomes the partial buffer
        float* pbuf = reinterpret_cast<float*>(smem + p.off_ring);  // [256 rows][8 tokens]
#pragma unroll
        for (int r = 0; r < RB_PER_WARP; ++r) {
            if (r < nvalid) {
                const int lr0 = (rbw0 + r) * TILE_ROWS + g, lr1 = lr0 + 8;
                *reinterpret_cast<float2*>(pbuf + lr0 * GEMV_MAX_M + 2 * t) = make_float2(tot[r][0], tot[r][1]);
                *reinterpret_cast<float2*>(pbuf + lr1 * GEMV_MAX_M + 2 * t) = make_float2(tot[r][2], tot[r][3]);
            }
        }
        cluster_sync_all();
        const int nrows_c = nrbv * TILE_ROWS;
        const uint32_t pbase = sbase + p.off_ring;
        if (a.glu) {
            // every CTA of the cluster sums and activates a slice of the outputs: output o of this 256-row block
            // has its gate sum in local row 32*(o/16) + o%16 and its up sum 16 rows further
            const int nout = nrows_c / 2;
            const int per_o = (nout + a.ksplit - 1) / a.ksplit;
            const int o_begin = split * per_o, o_end = min(nout, o_begin + per_o);
            const int nh = sg.n / 2;
            __half* ob = reinterpret_cast<__half*>(a.seg[0].out) + (size_t)row_base * nh;
            for (int i = threadIdx.x; i < (o_end - o_begin) * m_loc; i += blockDim.x) {
                const int o = o_begin + i / m_loc, tok = i % m_loc;
                const int lg = (o / TILE_ROWS) * 2 * TILE_ROWS + (o % TILE_ROWS), lu = lg + TILE_ROWS;
                float vg[8], vu[8];
#pragma unroll
                for (int s = 0; s < 8; ++s) {
                    vg[s] = s < a.ksplit ? ld_dsmem_f32(pbase + (uint32_t)(lg * GEMV_MAX_M + tok) * 4u, (unsigned)s) : 0.f;
                    vu[s] = s < a.ksplit ? ld_dsmem_f32(pbase + (uint32_t)(lu * GEMV_MAX_M + tok) * 4u, (unsigned)s) : 0.f;
                }
                float sg_ = 0.f, su = 0.f;
#pragma unroll
                for (int s = 0; s < 8; ++s) {
                    if (s < a.ksplit) {
                        sg_ += vg[s];
                        su += vu[s];
                    }
                }
                ob[(size_t)tok * nh + (rb_cta0 / 2) * TILE_ROWS + o] = silu_mul_f16(sg_, su);
            }
            cluster_sync_all();  // peers may still be reading this CTA's buffer
            if (stamp && threadIdx.x == 0) {
                stamp_now(5);
            }
            return;
        }
        const int per = (nrows_c + a.ksplit - 1) / a.ksplit;
        const int lr_begin = split * per, lr_end = min(nrows_c, lr_begin + per);
        for (int i = threadIdx.x; i < (lr_end - lr_begin) * m_loc; i += blockDim.x) {
            const int lr = lr_begin + i / m_loc, tok = i % m_loc;
            // all splits' loads first (a cluster has at most 8 CTAs), then the sum in split order
            float v[8];
#pragma unroll
            for (int s = 0; s < 8; ++s) {
                v[s] = s < a.ksplit ? ld_dsmem_f32(pbase + (uint32_t)(lr * GEMV_MAX_M + tok) * 4u, (unsigned)s) : 0.f;
            }
            float sum = 0.f;
#pragma unroll
            for (int s = 0; s < 8; ++s) {
                if (s < a.ksplit) {
                    sum += v[s];
                }
            }
            const int row = rb_cta0 * TILE_ROWS + lr;
            if (a.row_w != nullptr) {
                sum = mul_row_w(sum, a.row_w[row_base + tok]);
            }
            if (a.out_f16) {
                reinterpret_cast<__half*>(sg.out)[(size_t)tok * sg.n + row] = __float2half_rn(sum);
            } else {
                reinterpret_cast<float*>(sg.out)[(size_t)tok * sg.n + row] = sum;
            }
        }
        cluster_sync_all();  // peers may still be reading this CTA's buffer
        if (stamp && threadIdx.x == 0) {
            stamp_now(5);   // reduced and stored
        }
        return;
    }

    // split-K: park partials as part[split][cta][row_in_cta (256)][tok (8)], then the last CTA of
    // this column of the grid sums the splits in index order.
    float* mypart = a.part + ((size_t)split * gridDim.x + blockIdx.x) * (ROWS_PER_CTA * GEMV_MAX_M);
#pragma unroll
    for (int r = 0; r < RB_PER_WARP; ++r) {
        if (r < nvalid) {
            const int lr0 = (rbw0 + r) * TILE_ROWS + g, lr1 = lr0 + 8;
            *reinterpret_cast<float2*>(mypart + lr0 * GEMV_MAX_M + 2 * t) = make_float2(tot[r][0], tot[r][1]);
            *reinterpret_cast<float2*>(mypart + lr1 * GEMV_MAX_M + 2 * t) = make_float2(tot[r][2], tot[r][3]);
        }
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
    const int nrows = nrbv * TILE_ROWS;
    for (int i = threadIdx.x; i < ROWS_PER_CTA * (GEMV_MAX_M / 2); i += blockDim.x) {
        // one thread sums a (row, token pair): consecutive threads read consecutive float2
        const int lr = i / (GEMV_MAX_M / 2), tp = i % (GEMV_MAX_M / 2);
        if (lr < nrows && 2 * tp < m_loc) {
            const float* src = a.part + (size_t)blockIdx.x * (ROWS_PER_CTA * GEMV_MAX_M) + lr * GEMV_MAX_M + 2 * tp;
            const size_t stride = (size_t)gridDim.x * (ROWS_PER_CTA * GEMV_MAX_M);
            float2 sum = make_float2(0.f, 0.f);
#pragma unroll 8
            for (int s = 0; s < a.ksplit; ++s) {
                const float2 v = __ldcg(reinterpret_cast<const float2*>(src + s * stride));
                sum.x += v.x;
                sum.y += v.y;
            }
            const int row = rb_cta0 * TILE_ROWS + lr;
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                const int tok = 2 * tp + j;
                if (tok < m_loc) {
                    float v = j ? sum.y : sum.x;
                    if (a.row_w != nullptr) {
                        v = mul_row_w(v, a.row_w[row_base + tok]);
                    }
                    if (tp_on) {
                        tp_own_area(a.tp, s_seq)[(size_t)tok * a.tp.max_rows + row] = v;
                    } else if (a.out_f16) {
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
    if (tp_on) {
        tp_exchange(a, sg, rb_cta0, nrows, &s_seq, abort_flag, gridDim.x);
    }
    if (stamp && threadIdx.x == 0) {
        stamp_now(5);
    }
}

}  // namespace

int gemv_plan_ctas(GemvArgs& a) {
    int ctas = 0;
    for (int i = 0; i < a.nseg; ++i) {
        a.seg[i].cta0 = ctas;
        const int nrb = a.seg[i].n / TILE_ROWS;
        ctas += (nrb + CTA_RB - 1) / CTA_RB;
    }
    return ctas;
}

size_t gemv_smem_bytes(int k, int group, int m, int ksplit, int stages) {
    return (size_t)make_plan(k, group, m, ksplit, stages).total;
}

size_t gemv_part_floats(int grid_x, int ksplit) {
    return ksplit > 1 ? (size_t)ksplit * grid_x * (ROWS_PER_CTA * GEMV_MAX_M) : 0;
}

// Split-K policy (the reference sizes its split for a 70-SM part:
// crates/backend-gpu/src/rawcuda/w4a16_dec/kernels/decode.rs:3-20).  Measured on B200, one 256-row CTA cannot
// keep an SM's share of HBM busy but two to three resident CTAs can, and every extra split adds fixed cost,
// so the split aims at about 2.2 CTAs per SM, keeps at least two scale groups per split, stays within
// `max_split` (8 when the splits reduce inside a thread-block cluster) and within the shared-memory budget.
int gemv_pick_ksplit(int grid_x, int k, int group, int m, int sm_count, int max_split, int stages) {
    const int unit = group > TILE_K ? group : TILE_K;
    const int units = k / unit;
    int ks = (int)((2.2 * sm_count) / grid_x + 0.5);
    if (ks > max_split) {
        ks = max_split;
    }
    if (ks > units / 2) {
        ks = units / 2;
    }
    if (ks < 1) {
        ks = 1;
    }
    while (ks < units && gemv_smem_bytes(k, group, m, ks, stages) > (size_t)GEMV_SMEM_LIMIT) {
        ++ks;
    }
    return ks;
}

cudaError_t gemv_init_device() {
    cudaError_t e;
#define W4_SET(K) \
    e = cudaFuncSetAttribute(K, cudaFuncAttributeMaxDynamicSharedMemorySize, GEMV_SMEM_LIMIT); \
    if (e != cudaSuccess) return e;
    W4_SET((gemv_w4a16_kernel<128, true, 8>))
    W4_SET((gemv_w4a16_kernel<128, false, 8>))
    W4_SET((gemv_w4a16_kernel<32, true, 8>))
    W4_SET((gemv_w4a16_kernel<32, false, 8>))
    W4_SET((gemv_w4a16_kernel<128, true, 16>))
    W4_SET((gemv_w4a16_kernel<128, false, 16>))
    W4_SET((gemv_w4a16_kernel<32, true, 16>))
    W4_SET((gemv_w4a16_kernel<32, false, 16>))
#undef W4_SET
    return cudaSuccess;
}

template <int CW>
static cudaError_t launch_gemv_cw(const GemvArgs& a, const SmemPlan& p, cudaLaunchConfig_t& cfg) {
    cfg.blockDim = dim3((CW + 1) * 32);
    if (a.group == 128) {
        if (a.subnormal) {
            return cudaLaunchKernelEx(&cfg, gemv_w4a16_kernel<128, true, CW>, a, p);
        }
        return cudaLaunchKernelEx(&cfg, gemv_w4a16_kernel<128, false, CW>, a, p);
    }
    if (a.subnormal) {
        return cudaLaunchKernelEx(&cfg, gemv_w4a16_kernel<32, true, CW>, a, p);
    }
    return cudaLaunchKernelEx(&cfg, gemv_w4a16_kernel<32, false, CW>, a, p);
}

cudaError_t launch_gemv(const GemvArgs& a, int grid_x, cudaStream_t st) {
    const SmemPlan p = make_plan(a.k, a.group, a.m, a.ksplit, a.ring_stages);
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(grid_x, a.ksplit);
    cfg.dynamicSmemBytes = p.total;
    cfg.stream = st;
    cudaLaunchAttribute attr[2];
    int na = 0;
    if (a.pdl) {
        attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[na].val.programmaticStreamSerializationAllowed = 1;
        ++na;
    }
    if (a.cluster) {
        attr[na].id = cudaLaunchAttributeClusterDimension;
        attr[na].val.clusterDim.x = 1;
        attr[na].val.clusterDim.y = a.ksplit;  // grid.y == ksplit: one cluster per row block
        attr[na].val.clusterDim.z = 1;
        ++na;
    }
    cfg.attrs = attr;
    cfg.numAttrs = na;
    return a.cons_warps == 16 ? launch_gemv_cw<16>(a, p, cfg) : launch_gemv_cw<8>(a, p, cfg);
}

}  // namespace w4
