// Decode GEMV, "row block" form: a CTA owns ALL of K for 32 rows at a time, its warps split K.  Two kernels: the 8-warp
// one described first, which walks any number of units, and a 16-warp variant for launches whose units are all resident
// at once (further down).
//
// Same product and arithmetic as the other decode forms (crates/backend-gpu/src/rawcuda/assets/decode.cu:46-267 is
// what they replace): mma.sync m16n8k16 with the weight tile as the 16-row operand, the raw nibbles as exact f16
// subnormals, the zero point as the C operand of a group's first MMA, f32 accumulation per scale group and the f32
// group scale applied to the group's sum.  What differs is the shape of the work.  The persistent form deals equal
// K x row ranges to 296 CTAs and pays for it after the loop: row blocks shared between CTAs are parked in global
// memory, ticketed and summed by the last arriver -- a fence, an atomic and a round of loads, about 3 us per launch
// in which no weight byte moves.  Here nothing is shared between CTAs:
//   * a 16-row x 64-channel tile of the T64 layout is 512 contiguous bytes = one coalesced 16-byte load per lane, and
//     the tile of the next row block follows it in memory; so the weights need no shared-memory ring, no producer warp
//     and no barrier: each warp keeps four k-blocks of two row blocks (4 KB) in flight in registers and refills a slot
//     as soon as it has been multiplied, across the boundary from one pair of row blocks to the CTA's next one;
//   * the eight warps' partial sums meet in shared memory (double-buffered: one __syncthreads per 32 rows), no global
//     scratch, no ticket, no wait on any other CTA;
//   * the first four k-blocks of every warp are requested BEFORE griddepcontrol.wait: while the previous kernel of the
//     stream drains, the next one already has 32 KB per CTA on the way;
//   * what a warp multiplies after x has arrived is on the launch's critical path, and there the chain of MMAs on one
//     accumulator is what a warp waits for: a group's MMAs therefore alternate between two accumulators per row block
//     (added when the group closes), and the ring is four k-blocks deep, not six, to leave the registers for it
//     (qkv 7.7 -> 7.0 us, the gate_up shard of four GPUs 8.3 -> 7.3; four accumulators per row block were slower).
// What bounds it, measured on gate_up (89 MB) with parts of the kernel switched off: the arithmetic costs 5 us of 24 (at
// 16 warps per SM -- 128 registers per thread -- every warp issues one instruction in ten cycles), the wait for the
// previous kernel of the stream 3 us, staging x and the sums over the warps nothing; with all of it removed the kernel
// reads the matrix in 16.4 us, which is what a bare read loop with the same addresses and residency achieves (18.5 us
// at 16 warps per SM, 15.1 us at 32; a loop over 8 KB pieces in address order, the persistent form's pattern, 13.0 us).
// Variants with fewer registers (two or four k-blocks in flight, three or four CTAs per SM) spilled and were slower,
// 16-row units at four CTAs per SM were slower (more CTAs pay the prologue), prefetching the warp's next tiles into L2
// before the dependency wait gained 0.2 us.  Two variants that fed each warp's own shared-memory ring with copies
// instead were measured and dropped: one bulk copy per 1 KB tile pair (2.5 TB/s on gate_up: the copy engine's cost
// per copy) and one tensor-map copy per chunk of four k-blocks x two row blocks (3.0 TB/s).  So this form is chosen
// for launches of moderate size and K only (Dec::gemv_select), where the fixed cost of the persistent form weighs more
// than the streaming rate.
// The price is the activations: every CTA stages all of x (m x k f16) and its group sums in shared memory, from L2,
// once.  That bounds the form to small m; larger batches keep the other forms.
#include <cuda_fp16.h>

#include <algorithm>

#include "gemv_common.cuh"

namespace w4 {

namespace {

constexpr int RB_THREADS = 256;   // 8 warps
constexpr int RB_WARPS = RB_THREADS / 32;
constexpr int RB_MAXTOK = 4;
constexpr int RB_XPAD = 64;       // bytes added to a token's row of x so that the two tokens of a quarter-warp hit distinct banks
constexpr int RB_GROUP = 128;

// RBW = 16-row blocks per unit (2: a warp multiplies two neighbouring tiles with the same activation fragments, two
// CTAs per SM;  1: for matrices with fewer row blocks than SMs -- tensor-parallel shards --, so that more CTAs stream,
// three CTAs per SM).
// U = k-blocks in flight per warp (registers), of all RBW row blocks.
// TP: the fused all-reduce of a row-parallel shard (its own instantiation: the exchange costs registers).
template <int RBW, int RB_U, bool TP>
__global__ void __launch_bounds__(RB_THREADS, RBW == 2 ? 2 : 3) gemv_rb_kernel(const GemvArgs a, const int total_units) {
    extern __shared__ __align__(16) unsigned char smem[];
    __shared__ float red[2][RB_WARPS][RBW][TILE_ROWS][RB_MAXTOK];
    __shared__ __align__(16) uint32_t zero16[4];
    __shared__ unsigned s_seq;     // fused all-reduce: this launch's exchange number
    __shared__ int s_abort;

    // the next kernel of the stream may be scheduled as soon as this one is resident
    if (a.pdl) {
        asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    }
    // optional timeline (diagnostic; a.dbg is null in normal runs): wall-clock stamps of thread 0, recomputed from the
    // arguments at every site so that nothing stays in registers
    auto stamp_now = [&](int j) {
        if (a.dbg != nullptr && threadIdx.x == 0 && (int)blockIdx.x < DBG_CTAS) {
            unsigned long long ns;
            asm volatile("mov.u64 %0, %globaltimer;" : "=l"(ns));
            a.dbg[((size_t)a.dbg_seq * DBG_CTAS + blockIdx.x) * DBG_STAMPS + j] = (long long)ns;
        }
    };
    stamp_now(0);   // CTA entry; slots 0..5 as in the other forms (entry, dependency wait over, x staged, loop start, loop
                    // end, stored), 6 = SM id, 7 = units of this CTA, 8 = first tiles requested
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int ngroups = a.k / RB_GROUP;
    // this warp's groups [g0, g1) = k-blocks [2 g0, 2 g1), the same for every unit
    const int g0 = ngroups * warp / RB_WARPS, g1 = ngroups * (warp + 1) / RB_WARPS;
    const int kb0 = 2 * g0, nk = 2 * (g1 - g0);
    const int my_units = (int)blockIdx.x < total_units ? (total_units - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x : 0;
    const int S = my_units * nk;   // this warp's tiles pairs, in the order it multiplies them

    // One segment (the fused q|k|v and gate|up launches keep the other forms): this CTA's units are the row blocks
    // RBW * (blockIdx.x + j * gridDim.x), so a cursor moves from unit to unit by a constant stride.
    const GemvSeg& sg = a.seg[0];
    const int nrb = sg.n / TILE_ROWS;
    const size_t pitch = (size_t)nrb * 32;                                 // uint4 between k-blocks
    const int ustride = (int)gridDim.x * RBW;                              // row blocks between consecutive units of this CTA
    const int rb_first = (int)blockIdx.x * RBW;

    // ---- the register ring: position s = (unit s / nk, k-block kb0 + s % nk); cursors walk it without divisions ----
    struct Cursor {
        const uint4* p;         // next tile of the first row block
        const uint32_t* sp;     // next group's scale pair of the first row block
        int kin, rb;
        int off2;               // uint4 from the first row block's tile to the second's (0 when there is none: read twice)
        int soff2;              // the same for the scale pairs, in u32
    };
    auto cursor_offsets = [&](Cursor& c) {
        const bool second = RBW == 2 && c.rb + 1 < nrb;
        c.off2 = second ? 32 : 0;
        c.soff2 = second ? ngroups * 8 : 0;
    };
    auto cursor_init = [&](Cursor& c) {
        c.rb = rb_first;
        c.kin = 0;
        c.p = sg.qt + (size_t)c.rb * 32 + lane + (size_t)kb0 * pitch;
        c.sp = sg.st + ((size_t)c.rb * ngroups + g0) * 8 + g;
        cursor_offsets(c);
    };
    // End of a unit: back to the warp's first k-block, on to the CTA's next unit.  After the last unit the cursor walks
    // that unit again: the ring may always be refilled (a few tiles are read twice at the very end, nothing is read
    // out of range) and the hot loop needs no test for the end.
    auto cursor_next_unit = [&](Cursor& c, bool weights) {
        if (weights) {
            c.p -= (size_t)nk * pitch;
        } else {
            c.sp -= (size_t)(nk / 2) * 8;
        }
        if (c.rb + ustride < nrb) {
            c.rb += ustride;
            c.p += (size_t)ustride * 32;
            c.sp += (size_t)ustride * ngroups * 8;
            cursor_offsets(c);
        }
        c.kin = 0;
    };
    uint4 wq[RB_U][RBW];
    uint32_t sq[RB_U / 2][RBW];
    Cursor fw{}, fs{};          // where the next weight tile / the next scale pair is fetched from
    auto fetch = [&](uint4 (&w)[RBW]) {
        w[0] = __ldg(fw.p);
        if (RBW == 2) {
            w[RBW - 1] = __ldg(fw.p + fw.off2);
        }
        fw.p += pitch;
        if (++fw.kin == nk) {
            cursor_next_unit(fw, true);
        }
    };
    auto fetch_scale = [&](uint32_t (&sc)[RBW]) {
        sc[0] = __ldg(fs.sp);
        if (RBW == 2) {
            sc[RBW - 1] = __ldg(fs.sp + fs.soff2);
        }
        fs.sp += 8;
        fs.kin += 2;
        if (fs.kin == nk) {
            cursor_next_unit(fs, false);
        }
    };
    if (my_units == 0) {
        return;                 // more CTAs than units never happens (the grid is at most the unit count)
    }
    if (a.dbg != nullptr && threadIdx.x == 0 && (int)blockIdx.x < DBG_CTAS) {
        unsigned smid;
        asm volatile("mov.u32 %0, %smid;" : "=r"(smid));
        long long* d = a.dbg + ((size_t)a.dbg_seq * DBG_CTAS + blockIdx.x) * DBG_STAMPS;
        d[6] = smid;
        d[7] = my_units;
    }
    cursor_init(fw);
    cursor_init(fs);
    if (nk > 0) {               // a warp without a group (fewer groups than warps) only takes part in the sums
#pragma unroll
        for (int u = 0; u < RB_U; ++u) {
            fetch(wq[u]);
        }
#pragma unroll
        for (int u = 0; u < RB_U / 2; ++u) {
            fetch_scale(sq[u]);
        }
    }

    // ---- x may be the previous kernel's output: only now wait for it; stage it and its group sums --------------
    stamp_now(8);   // first tiles requested
    if (a.pdl) {
        asm volatile("griddepcontrol.wait;" ::: "memory");
    }
    stamp_now(1);   // the previous kernel of the stream is complete
    if (threadIdx.x < 4) {
        zero16[threadIdx.x] = 0;
    }
    constexpr bool tp_on = TP;
    if (threadIdx.x == 0) {
        // read only now: the previous launch advances the number as it ends
        s_seq = tp_on ? *reinterpret_cast<volatile unsigned*>(a.tp.seq) + 1u : 0u;
        s_abort = 0;
    }
    const int xstride = a.k * 2 + RB_XPAD;
    float* zs = reinterpret_cast<float*>(smem + (size_t)a.m * xstride);   // [group][4 tokens]: -8 * 2^-24 * sum of x
    {
        const int per_tok = a.k / 8;                                       // 16-byte pieces per token (16 per group)
        const int total = a.m * per_tok;
        const uint4* xg = reinterpret_cast<const uint4*>(a.x);
        // four loads per thread are requested before the first is used: the copy is a chain of L2 round trips otherwise
        constexpr int XB = 4;
        for (int i0 = 0; i0 < total; i0 += XB * RB_THREADS) {
            uint4 xr[XB];
#pragma unroll
            for (int b = 0; b < XB; ++b) {
                const int i = i0 + b * RB_THREADS + (int)threadIdx.x;
                xr[b] = i < total ? __ldg(xg + i) : make_uint4(0, 0, 0, 0);
            }
#pragma unroll
            for (int b = 0; b < XB; ++b) {
                const int i = i0 + b * RB_THREADS + (int)threadIdx.x;
                const bool live = i < total;
                const uint4 u = xr[b];
                int tok = 0, c = 0;
                if (live) {
                    tok = i / per_tok;
                    c = i - tok * per_tok;
                    *reinterpret_cast<uint4*>(smem + (size_t)tok * xstride + (size_t)c * 16) = u;
                }
                const float2 f0 = __half22float2(*reinterpret_cast<const __half2*>(&u.x));
                const float2 f1 = __half22float2(*reinterpret_cast<const __half2*>(&u.y));
                const float2 f2 = __half22float2(*reinterpret_cast<const __half2*>(&u.z));
                const float2 f3 = __half22float2(*reinterpret_cast<const __half2*>(&u.w));
                float v = ((f0.x + f0.y) + (f1.x + f1.y)) + ((f2.x + f2.y) + (f3.x + f3.y));
                // the 16 pieces of a group sit in 16 consecutive lanes
#pragma unroll
                for (int off = 8; off > 0; off >>= 1) {
                    v += __shfl_xor_sync(0xffffffffu, v, off);
                }
                if (live && (lane & 15) == 0) {
                    zs[(c >> 4) * RB_MAXTOK + tok] = -8.f * v * 5.9604644775390625e-08f;   // 2^-24
                }
            }
        }
        // tokens that do not exist contribute nothing
        for (int i = threadIdx.x; i < ngroups * RB_MAXTOK; i += RB_THREADS) {
            if ((i & (RB_MAXTOK - 1)) >= a.m) {
                zs[i] = 0.f;
            }
        }
    }
    __syncthreads();
    stamp_now(2);   // x and its group sums staged
    stamp_now(3);

    // lanes whose MMA column holds no token read 16 zero bytes, with stride 0: no branch in the loop
    const bool tok_lane = g < a.m;
    const unsigned char* xl = tok_lane ? smem + (size_t)g * xstride + t * 16 : reinterpret_cast<const unsigned char*>(zero16);
    const int xk = tok_lane ? 128 : 0, xh = tok_lane ? 64 : 0;
    // zero-point sums of tokens 2t, 2t+1 (lanes t >= 2 hold no token below five tokens: zeros, stride 0)
    const float* zl = t < RB_MAXTOK / 2 ? zs + 2 * t : reinterpret_cast<const float*>(zero16);
    const int zk = t < RB_MAXTOK / 2 ? RB_MAXTOK : 0;
    float tot[RBW][4];
#pragma unroll
    for (int r = 0; r < RBW; ++r) {
        tot[r][0] = tot[r][1] = tot[r][2] = tot[r][3] = 0.f;
    }
    int units_done = 0;
    int crb = rb_first;                                                    // first row block of the unit being multiplied
    // ---- a unit is complete in this warp: the eight warps' sums meet in shared memory -------------------------------
    auto flush_unit = [&]() {
        const int buf = units_done & 1;
        if (t < RB_MAXTOK / 2) {
#pragma unroll
            for (int r = 0; r < RBW; ++r) {
                // nibble units -> values: 2^24 for rows g, 2^20 for rows g+8
                red[buf][warp][r][g][2 * t] = tot[r][0] * 16777216.f;
                red[buf][warp][r][g][2 * t + 1] = tot[r][1] * 16777216.f;
                red[buf][warp][r][g + 8][2 * t] = tot[r][2] * 1048576.f;
                red[buf][warp][r][g + 8][2 * t + 1] = tot[r][3] * 1048576.f;
            }
        }
#pragma unroll
        for (int r = 0; r < RBW; ++r) {
            tot[r][0] = tot[r][1] = tot[r][2] = tot[r][3] = 0.f;
        }
        __syncthreads();
        if ((int)threadIdx.x < RBW * TILE_ROWS * a.m) {
            const int tok = (int)threadIdx.x / (RBW * TILE_ROWS), r32 = (int)threadIdx.x % (RBW * TILE_ROWS);
            const int r = r32 / TILE_ROWS, row = r32 % TILE_ROWS;
            if (crb + r < nrb) {
                float v = 0.f;
#pragma unroll
                for (int w = 0; w < RB_WARPS; ++w) {
                    v += red[buf][w][r][row][tok];                         // fixed order: the same bits every run
                }
                v *= sg.out_mul;
                const size_t o = (size_t)tok * sg.n + (size_t)(crb + r) * TILE_ROWS + row;
                if (tp_on) {
                    // row-parallel shard: the local sum goes to this rank's slot, the exchange below adds the peers'
                    tp_own_area(a.tp, s_seq)[(size_t)tok * a.tp.max_rows + (size_t)(crb + r) * TILE_ROWS + row] = v;
                } else if (a.out_f16) {
                    reinterpret_cast<__half*>(sg.out)[o] = __float2half_rn(v);
                } else {
                    reinterpret_cast<float*>(sg.out)[o] = v;
                }
            }
        }
        if (tp_on) {
            // all threads: push the unit's sums to every peer, wait (bounded) for theirs, add, store
            tp_exchange(a, sg, crb, min(RBW, nrb - crb) * TILE_ROWS, &s_seq, &s_abort, (unsigned)total_units);
        }
        ++units_done;
        crb += ustride;
    };
    if (nk == 0) {
        // fewer groups than warps: this warp adds zeros, once per unit, so that the CTA's barriers stay matched
        for (int j = 0; j < my_units; ++j) {
            flush_unit();
        }
        return;
    }
    int kin = 0;                                                           // k-block (inside the warp's range) being multiplied
    for (int base = 0; base < S; base += RB_U) {
#pragma unroll
        for (int u = 0; u < RB_U; u += 2) {
            const int s = base + u;
            if (s < S) {                                                   // warp-uniform: a whole group or nothing
                const int grp = g0 + kin / 2;
                // zero-point term of this group: (tokens 2t, 2t+1) x (rows g: 2^-24 per nibble unit, rows g+8: 2^-20)
                const float2 z = *reinterpret_cast<const float2*>(zl + grp * zk);
                // two accumulator chains per row block (words x, z and words y, w): consecutive MMAs of a chain are four
                // MMAs apart instead of two
                float cg[RBW][4], ch[RBW][4];
#pragma unroll
                for (int r = 0; r < RBW; ++r) {
                    cg[r][0] = z.x;
                    cg[r][1] = z.y;
                    cg[r][2] = 16.f * z.x;
                    cg[r][3] = 16.f * z.y;
                    ch[r][0] = ch[r][1] = ch[r][2] = ch[r][3] = 0.f;
                }
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    const int kb = kb0 + kin + h;
                    uint4 wv[RBW];
#pragma unroll
                    for (int r = 0; r < RBW; ++r) {
                        wv[r] = wq[u + h][r];
                    }
                    fetch(wq[u + h]);                                      // refill the slot at once
                    // word 2p+q of the lane holds rows g, g+8 at channels 32p + 8t + 4q + {0..3}: the activations of
                    // the same channels are 8 consecutive f16 at 8t (p = 0) and at 32 + 8t (p = 1)
                    const uint4 x0 = *reinterpret_cast<const uint4*>(xl + kb * xk);
                    const uint4 x1 = *reinterpret_cast<const uint4*>(xl + kb * xk + xh);
                    uint32_t af[4];
#pragma unroll
                    for (int r = 0; r < RBW; ++r) {
                        nibbles_as_subnormals(wv[r].x, af);
                        mma16816(cg[r], af, x0.x, x0.y);
                    }
#pragma unroll
                    for (int r = 0; r < RBW; ++r) {
                        nibbles_as_subnormals(wv[r].y, af);
                        mma16816(ch[r], af, x0.z, x0.w);
                    }
#pragma unroll
                    for (int r = 0; r < RBW; ++r) {
                        nibbles_as_subnormals(wv[r].z, af);
                        mma16816(cg[r], af, x1.x, x1.y);
                    }
#pragma unroll
                    for (int r = 0; r < RBW; ++r) {
                        nibbles_as_subnormals(wv[r].w, af);
                        mma16816(ch[r], af, x1.z, x1.w);
                    }
                }
#pragma unroll
                for (int r = 0; r < RBW; ++r) {
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        cg[r][i] += ch[r][i];
                    }
                }
                uint32_t s2[RBW];
#pragma unroll
                for (int r = 0; r < RBW; ++r) {
                    s2[r] = sq[u / 2][r];
                }
                fetch_scale(sq[u / 2]);
#pragma unroll
                for (int r = 0; r < RBW; ++r) {
                    const float2 sf = __half22float2(*reinterpret_cast<const __half2*>(&s2[r]));
                    tot[r][0] = fmaf(cg[r][0], sf.x, tot[r][0]);
                    tot[r][1] = fmaf(cg[r][1], sf.x, tot[r][1]);
                    tot[r][2] = fmaf(cg[r][2], sf.y, tot[r][2]);
                    tot[r][3] = fmaf(cg[r][3], sf.y, tot[r][3]);
                }
                if (kin + 2 == nk) {
                    flush_unit();
                    kin = 0;
                } else {
                    kin += 2;
                }
            }
        }
    }
    stamp_now(4);
    stamp_now(5);   // warp 0 is through its last unit (sums stored)
}

// ---- "unit" variant: one unit of 32 rows per CTA, 16 warps ----------------------------------------------------------
// For launches whose units all fit on the chip at once (at most two CTAs per SM): qkv, o_proj, every tensor-parallel
// shard.  Such a launch lasts as long as its fullest SM, and an SM with one or two 8-warp CTAs of 128 registers is
// latency-bound in what it multiplies after x has arrived.  Here K is split over 16 warps, and the weights do not wait
// in registers: a warp's first group is loaded into registers and all its other groups (and its scales) go to shared
// memory by asynchronous copies, all requested before the dependency wait.  What is left after the wait is x, the
// arithmetic out of shared memory with 32 warps per SM at 64 registers, and the sum over the warps.
constexpr int RU_WARPS = 16;
constexpr int RU_THREADS = RU_WARPS * 32;

template <bool TP>
__global__ void __launch_bounds__(RU_THREADS, 2) gemv_ru_kernel(const GemvArgs a, const int total_units) {
    extern __shared__ __align__(16) unsigned char smem[];   // x rows, group sums | weight slab | scale words
    __shared__ float red[RU_WARPS][2][TILE_ROWS][RB_MAXTOK];
    __shared__ __align__(16) uint32_t zero16[4];
    __shared__ unsigned s_seq;
    __shared__ int s_abort;
    if (a.pdl) {
        asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    }
    auto stamp_now = [&](int j) {
        if (a.dbg != nullptr && threadIdx.x == 0 && (int)blockIdx.x < DBG_CTAS) {
            unsigned long long ns;
            asm volatile("mov.u64 %0, %globaltimer;" : "=l"(ns));
            a.dbg[((size_t)a.dbg_seq * DBG_CTAS + blockIdx.x) * DBG_STAMPS + j] = (long long)ns;
        }
    };
    stamp_now(0);   // same slots as the other forms: 6 = SM id, 7 = units of this CTA (one), 8 = first tiles requested
    if (a.dbg != nullptr && threadIdx.x == 0 && (int)blockIdx.x < DBG_CTAS) {
        unsigned smid;
        asm volatile("mov.u32 %0, %smid;" : "=r"(smid));
        long long* d = a.dbg + ((size_t)a.dbg_seq * DBG_CTAS + blockIdx.x) * DBG_STAMPS;
        d[6] = smid;
        d[7] = 1;
    }
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int ngroups = a.k / RB_GROUP;
    const int g0 = ngroups * warp / RU_WARPS, g1 = ngroups * (warp + 1) / RU_WARPS;
    const int ng = g1 - g0;
    const GemvSeg& sg = a.seg[0];
    const int nrb = sg.n / TILE_ROWS;
    const size_t pitch = (size_t)nrb * 32;
    const int rb = (int)blockIdx.x * 2;
    const bool second = rb + 1 < nrb;
    const int off2 = second ? 32 : 0, soff2 = second ? ngroups * 8 : 0;
    // groups kept in shared memory by the warps before this one: every warp with a group keeps one in registers
    const int stored_before = ngroups >= RU_WARPS ? g0 - warp : 0;   // below 16 groups no warp has a second one
    const uint32_t sbase = smem_u32(smem);
    const uint32_t slab = sbase + (uint32_t)a.rb_stash + (uint32_t)stored_before * 2048u + (uint32_t)lane * 16u;
    const uint32_t scb = sbase + (uint32_t)a.rb_stash2;
    uint4 wq[2][2];
    if (ng > 0) {
        const uint4* p = sg.qt + ((size_t)(2 * g0) * nrb + rb) * 32 + lane;
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            wq[h][0] = __ldg(p + h * pitch);
            wq[h][1] = __ldg(p + h * pitch + off2);
        }
        p += 2 * pitch;
        for (int j = 1; j < ng; ++j) {
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const uint32_t dst = slab + (uint32_t)((j - 1) * 2 + h) * 1024u;
                cp_async_16(dst, p + h * pitch);
                cp_async_16(dst + 512u, p + h * pitch + off2);
            }
            p += 2 * pitch;
        }
        // scale words of rows g / g+8: [group][row block][8], 16 lanes per group
        if (lane < 16) {
            const int r = lane >> 3, gi = lane & 7;
            const uint32_t* sp = sg.st + ((size_t)rb * ngroups + g0) * 8 + (r ? soff2 : 0) + gi;
            for (int j = 0; j < ng; ++j) {
                cp_async_4(scb + (uint32_t)(((g0 + j) * 2 + r) * 8 + gi) * 4u, sp + (size_t)j * 8);
            }
        }
    }
    stamp_now(8);
    if (a.pdl) {
        asm volatile("griddepcontrol.wait;" ::: "memory");
    }
    stamp_now(1);
    if (threadIdx.x < 4) {
        zero16[threadIdx.x] = 0;
    }
    if (threadIdx.x == 0) {
        s_seq = TP ? *reinterpret_cast<volatile unsigned*>(a.tp.seq) + 1u : 0u;
        s_abort = 0;
    }
    const int xstride = a.k * 2 + RB_XPAD;
    float* zs = reinterpret_cast<float*>(smem + (size_t)a.m * xstride);
    {
        const int per_tok = a.k / 8;
        const int total = a.m * per_tok;
        const uint4* xg = reinterpret_cast<const uint4*>(a.x);
        constexpr int XB = 2;
        for (int i0 = 0; i0 < total; i0 += XB * RU_THREADS) {
            uint4 xr[XB];
#pragma unroll
            for (int b = 0; b < XB; ++b) {
                const int i = i0 + b * RU_THREADS + (int)threadIdx.x;
                xr[b] = i < total ? __ldg(xg + i) : make_uint4(0, 0, 0, 0);
            }
#pragma unroll
            for (int b = 0; b < XB; ++b) {
                const int i = i0 + b * RU_THREADS + (int)threadIdx.x;
                const bool live = i < total;
                const uint4 u = xr[b];
                int tok = 0, c = 0;
                if (live) {
                    tok = i / per_tok;
                    c = i - tok * per_tok;
                    *reinterpret_cast<uint4*>(smem + (size_t)tok * xstride + (size_t)c * 16) = u;
                }
                const float2 f0 = __half22float2(*reinterpret_cast<const __half2*>(&u.x));
                const float2 f1 = __half22float2(*reinterpret_cast<const __half2*>(&u.y));
                const float2 f2 = __half22float2(*reinterpret_cast<const __half2*>(&u.z));
                const float2 f3 = __half22float2(*reinterpret_cast<const __half2*>(&u.w));
                float v = ((f0.x + f0.y) + (f1.x + f1.y)) + ((f2.x + f2.y) + (f3.x + f3.y));
#pragma unroll
                for (int off = 8; off > 0; off >>= 1) {
                    v += __shfl_xor_sync(0xffffffffu, v, off);
                }
                if (live && (lane & 15) == 0) {
                    zs[(c >> 4) * RB_MAXTOK + tok] = -8.f * v * 5.9604644775390625e-08f;
                }
            }
        }
        for (int i = threadIdx.x; i < ngroups * RB_MAXTOK; i += RU_THREADS) {
            if ((i & (RB_MAXTOK - 1)) >= a.m) {
                zs[i] = 0.f;
            }
        }
    }
    cp_async_wait_all();        // weights: each lane reads back what it copied; scales: other lanes' copies -> the barrier
    __syncthreads();
    stamp_now(2);
    stamp_now(3);

    const bool tok_lane = g < a.m;
    const unsigned char* xl = tok_lane ? smem + (size_t)g * xstride + t * 16 : reinterpret_cast<const unsigned char*>(zero16);
    const int xk = tok_lane ? 128 : 0, xh = tok_lane ? 64 : 0;
    const float* zl = t < RB_MAXTOK / 2 ? zs + 2 * t : reinterpret_cast<const float*>(zero16);
    const int zk = t < RB_MAXTOK / 2 ? RB_MAXTOK : 0;
    float tot[2][4];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        tot[r][0] = tot[r][1] = tot[r][2] = tot[r][3] = 0.f;
    }
    // one scale group (two k-blocks) of both row blocks: w[h][r] = the lane's 16 bytes of tile (k-block h, row block r)
    auto do_group = [&](int grp, const uint4 (&w)[2][2]) {
        const float2 z = *reinterpret_cast<const float2*>(zl + grp * zk);
        float cg[2][4];
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            cg[r][0] = z.x;
            cg[r][1] = z.y;
            cg[r][2] = 16.f * z.x;
            cg[r][3] = 16.f * z.y;
        }
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int kb = 2 * grp + h;
            const uint4 x0 = *reinterpret_cast<const uint4*>(xl + kb * xk);
            const uint4 x1 = *reinterpret_cast<const uint4*>(xl + kb * xk + xh);
            uint32_t af[4];
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                nibbles_as_subnormals(w[h][r].x, af);
                mma16816(cg[r], af, x0.x, x0.y);
            }
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                nibbles_as_subnormals(w[h][r].y, af);
                mma16816(cg[r], af, x0.z, x0.w);
            }
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                nibbles_as_subnormals(w[h][r].z, af);
                mma16816(cg[r], af, x1.x, x1.y);
            }
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                nibbles_as_subnormals(w[h][r].w, af);
                mma16816(cg[r], af, x1.z, x1.w);
            }
        }
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            const uint32_t s2 = lds32(scb + (uint32_t)((grp * 2 + r) * 8 + g) * 4u);
            const float2 sf = __half22float2(*reinterpret_cast<const __half2*>(&s2));
            tot[r][0] = fmaf(cg[r][0], sf.x, tot[r][0]);
            tot[r][1] = fmaf(cg[r][1], sf.x, tot[r][1]);
            tot[r][2] = fmaf(cg[r][2], sf.y, tot[r][2]);
            tot[r][3] = fmaf(cg[r][3], sf.y, tot[r][3]);
        }
    };
    if (ng > 0) {
        do_group(g0, wq);
        for (int j = 1; j < ng; ++j) {
            uint4 w[2][2];
#pragma unroll
            for (int h = 0; h < 2; ++h) {
#pragma unroll
                for (int r = 0; r < 2; ++r) {
                    w[h][r] = lds128(slab + (uint32_t)((j - 1) * 2 + h) * 1024u + (uint32_t)r * 512u);
                }
            }
            do_group(g0 + j, w);
        }
    }
    stamp_now(4);
    if (t < RB_MAXTOK / 2) {
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            red[warp][r][g][2 * t] = tot[r][0] * 16777216.f;
            red[warp][r][g][2 * t + 1] = tot[r][1] * 16777216.f;
            red[warp][r][g + 8][2 * t] = tot[r][2] * 1048576.f;
            red[warp][r][g + 8][2 * t + 1] = tot[r][3] * 1048576.f;
        }
    }
    __syncthreads();
    if ((int)threadIdx.x < 2 * TILE_ROWS * a.m) {
        const int tok = (int)threadIdx.x / (2 * TILE_ROWS), r32 = (int)threadIdx.x % (2 * TILE_ROWS);
        const int r = r32 / TILE_ROWS, row = r32 % TILE_ROWS;
        if (rb + r < nrb) {
            float v = 0.f;
#pragma unroll
            for (int w = 0; w < RU_WARPS; ++w) {
                v += red[w][r][row][tok];                                  // fixed order: the same bits every run
            }
            v *= sg.out_mul;
            const size_t o = (size_t)tok * sg.n + (size_t)(rb + r) * TILE_ROWS + row;
            if (TP) {
                tp_own_area(a.tp, s_seq)[(size_t)tok * a.tp.max_rows + (size_t)(rb + r) * TILE_ROWS + row] = v;
            } else if (a.out_f16) {
                reinterpret_cast<__half*>(sg.out)[o] = __float2half_rn(v);
            } else {
                reinterpret_cast<float*>(sg.out)[o] = v;
            }
        }
    }
    if (TP) {
        tp_exchange(a, sg, rb, min(2, nrb - rb) * TILE_ROWS, &s_seq, &s_abort, (unsigned)total_units);
    }
    stamp_now(5);
}

}  // namespace

cudaError_t gemv_rb_init_device() {
    cudaError_t e = cudaFuncSetAttribute(gemv_rb_kernel<2, 4, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024);
    if (e == cudaSuccess) {
        e = cudaFuncSetAttribute(gemv_rb_kernel<2, 4, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024);
    }
    if (e == cudaSuccess) {
        e = cudaFuncSetAttribute(gemv_rb_kernel<1, 6, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 72 * 1024);
    }
    if (e == cudaSuccess) {
        e = cudaFuncSetAttribute(gemv_rb_kernel<1, 6, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 72 * 1024);
    }
    if (e == cudaSuccess) {
        e = cudaFuncSetAttribute(gemv_ru_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024);
    }
    if (e == cudaSuccess) {
        e = cudaFuncSetAttribute(gemv_ru_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024);
    }

    return e;
}

static size_t gemv_rb_smem(const GemvArgs& a) {
    return (size_t)a.m * ((size_t)a.k * 2 + RB_XPAD) + (size_t)(a.k / RB_GROUP) * RB_MAXTOK * sizeof(float);
}

// Whether the row-block form can take this call: one segment, 128-channel groups, at most four tokens, x small enough for two CTAs per SM.
bool gemv_rb_fits(const GemvArgs& a) {
    return a.nseg == 1 && a.group == RB_GROUP && a.m >= 1 && a.m <= RB_MAXTOK && a.k % RB_GROUP == 0 && a.k / RB_GROUP >= 1 &&
           gemv_rb_smem(a) <= (size_t)100 * 1024;
}

// Shared memory of the 16-warp variant: x and its group sums, the groups beyond each warp's first, the scale words.
static size_t gemv_ru_smem(const GemvArgs& a, int* off_slab, int* off_sc) {
    const int ngroups = a.k / RB_GROUP;
    size_t off = ((size_t)a.m * ((size_t)a.k * 2 + RB_XPAD) + (size_t)ngroups * RB_MAXTOK * sizeof(float) + 15) & ~(size_t)15;
    *off_slab = (int)off;
    off += (size_t)(ngroups > RU_WARPS ? ngroups - RU_WARPS : 0) * 2048;
    *off_sc = (int)off;
    off += (size_t)ngroups * 2 * 8 * 4;
    return off;
}

// The 16-warp variant takes a call whose 32-row units are all resident at once, two CTAs per SM.
bool gemv_ru_fits(const GemvArgs& a, int sm_count) {
    int o1, o2;
    return !a.rb_no_units && gemv_rb_fits(a) && (a.seg[0].n / TILE_ROWS + 1) / 2 <= 2 * sm_count &&
           gemv_ru_smem(a, &o1, &o2) <= (size_t)100 * 1024;
}

// Units over all segments (seg[].cta0 = first unit of the segment) and the row blocks per unit: two for the 16-warp
// variant and for matrices with more row blocks than SMs, else one (more CTAs, more loads in flight).
int gemv_rb_plan(GemvArgs& a, int sm_count, int& rbw) {
    int nrb = 0;
    for (int i = 0; i < a.nseg; ++i) {
        nrb += a.seg[i].n / TILE_ROWS;
    }
    rbw = (!gemv_ru_fits(a, sm_count) && nrb <= sm_count && gemv_rb_smem(a) <= (size_t)72 * 1024) ? 1 : 2;
    int total = 0;
    for (int i = 0; i < a.nseg; ++i) {
        a.seg[i].cta0 = total;
        total += (a.seg[i].n / TILE_ROWS + rbw - 1) / rbw;
    }
    return total;
}

// Which kernel a row-block launch runs (also what the library reports as the last kernel's name).
const char* gemv_rb_variant(const GemvArgs& a, int total_units, int rbw, int sm_count) {
    if (rbw == 2 && gemv_ru_fits(a, sm_count)) {
        return "gemv_ru_kernel";
    }
    return rbw == 2 ? "gemv_rb_kernel<2>" : "gemv_rb_kernel<1>";
}

cudaError_t launch_gemv_rb(const GemvArgs& a_in, int total_units, int rbw, int sm_count, cudaStream_t st) {
    GemvArgs a = a_in;
    cudaLaunchConfig_t cfg{};
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
    const char variant = gemv_rb_variant(a, total_units, rbw, sm_count)[6];
    if (variant == 'u') {
        cfg.gridDim = dim3(total_units);
        cfg.blockDim = dim3(RU_THREADS);
        cfg.dynamicSmemBytes = gemv_ru_smem(a, &a.rb_stash, &a.rb_stash2);
        return a.tp.world > 1 ? cudaLaunchKernelEx(&cfg, gemv_ru_kernel<true>, a, total_units)
                              : cudaLaunchKernelEx(&cfg, gemv_ru_kernel<false>, a, total_units);
    }

    cfg.gridDim = dim3(std::min(total_units, (rbw == 2 ? 2 : 3) * sm_count));
    cfg.blockDim = dim3(RB_THREADS);
    cfg.dynamicSmemBytes = gemv_rb_smem(a);
    if (a.tp.world > 1) {
        return rbw == 2 ? cudaLaunchKernelEx(&cfg, gemv_rb_kernel<2, 4, true>, a, total_units)
                        : cudaLaunchKernelEx(&cfg, gemv_rb_kernel<1, 6, true>, a, total_units);
    }
    return rbw == 2 ? cudaLaunchKernelEx(&cfg, gemv_rb_kernel<2, 4, false>, a, total_units)
                    : cudaLaunchKernelEx(&cfg, gemv_rb_kernel<1, 6, false>, a, total_units);
}

}  // namespace w4
