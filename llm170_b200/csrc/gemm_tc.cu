// Prefill W4A16 GEMM on the 5th-generation tensor cores:  y[m][n] = sum_k x[m][k] * f16((q[n][k]-8)*s[n][k/g]).
//
// Takes the place of the reference's prefill GEMMs (vendored Marlin instantiations launched from
// crates/backend-gpu/src/rawcuda/w4a16_dec/kernels/marlin.rs:94-213, and the hand-written
// crates/backend-gpu/src/rawcuda/assets/moe.cu:1139-1587 / gptq4.cu:984-1147), which are mma.sync kernels.
// Like them it multiplies the dequantised weight ROUNDED ONCE TO F16 (hmul2 of the exact integer and
// the f16 scale; the reference's own model of this is crates/server/src/probes/w4a16/gpu/bench.rs:240)
// and accumulates in f32.
//
// One CTA computes a 128 (tokens) x 256 (weight rows) tile:
//   warp 0      producer: TMA-loads the f16 activation tile (128 x 64, 128B swizzle) and bulk-copies the
//               raw int4 tiles (16 x 512 B of the T64 layout) of each 64-wide k-block into a 6-stage ring
//   warps 2-17  expand int4 -> f16 into a 2-stage ring of K-major 128B-swizzled B operands (one 16-byte
//               chunk = 8 consecutive k of one weight row), then signal the MMA warp
//   warp 1      one lane issues 4 x tcgen05.mma (M128 N256 K16, f16 x f16 -> f32 in TMEM) per k-block and
//               commits the stage back to the producer
//   warps 2-17  epilogue: tcgen05.ld the f32 accumulators (each warp its TMEM lane quadrant, every fourth
//               32-column chunk), convert, store y
// Every mbarrier wait is bounded: on expiry the kernel records a status code, all roles fall through to
// the common exit, TMEM is released, and the host reports an error instead of hanging.
#include <cuda.h>
#include <cuda_fp16.h>

#include <algorithm>
#include <string>

#include "../../include/w4a16_b200.h"
#include "dec.h"
#include "ptx.cuh"

namespace w4 {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

namespace {

constexpr int BM = 128;           // tokens per tile (UMMA M)
constexpr int BN = 256;           // weight rows per tile (UMMA N)
constexpr int BK = TILE_K;        // 64 k per stage = one 128-byte swizzle row of f16
constexpr int A_BYTES = BM * BK * 2;          // 16 KB per 128-token block
constexpr int RAW_BYTES = BN * BK / 2;        // 8 KB
constexpr int B_BYTES = BN * BK * 2;          // 32 KB
constexpr int NUM_DQ_WARPS = 16;   // one 16-row block of the tile each
constexpr int NUM_THREADS = (2 + NUM_DQ_WARPS) * 32;
// MT = 128-token blocks per CTA tile (1 or 2).  With MT = 2 one expanded weight stage feeds two MMAs groups
// (two TMEM accumulators), halving the expand work and the shared-memory traffic per flop.
template <int MT> struct Cfg {
    static constexpr int NT = MT == 1 ? 6 : 4;   // TMA ring: activation blocks + raw int4 tile per stage
    static constexpr int NB = 2;                 // ring of expanded f16 weight tiles (3 with a shallower TMA ring measured slower)
    static constexpr int A_STAGE = MT * A_BYTES;
    static constexpr int TMEM_COLS = 256 * MT;
    static constexpr int SMEM = NT * (A_STAGE + RAW_BYTES) + NB * B_BYTES + 1024 /* alignment slack */ + 256 /* barriers */;
};
constexpr int GROUP_M = 8;        // m-tiles per rasterisation group (L2 reuse of the weight tiles)

struct GemmArgs {
    const uint32_t* qt;
    const uint32_t* st;  // scale pairs
    void* out;
    int m, n, k;
    int out_f16;
    int m_tiles, n_tiles;
    int nrb_w;       // 16-row blocks of the resident weight matrix (= n/16; experts stacked along n when grouped)
    // grouped (MoE) mode: m-tiles come from a device table, one expert's weights per tile
    int grouped;
    const int* tile_expert;
    const int* tile_row0;
    const int* tile_rows;
    const int* num_tiles;
    int expert0;          // first expert held by this decoder
    const float* row_w;   // optional per-row factor applied in the epilogue (routing weight)
    float out_mul;        // power of two applied to every sum (undoes the shift of bf16 scales; normally 1)
    int glu;              // 1: weight rows are interleaved gate / up 16-row blocks; the epilogue stores
                          // f16(silu(f16 gate) * f16 up), n/2 values per row
    // split-K: the first `n_whole` tiles (in launch order) are one CTA each; every later tile is `ksplit` CTAs, each
    // multiplying k-blocks [nkb*s/ksplit, nkb*(s+1)/ksplit).  Their f32 partial tiles go to `part`, and the last
    // split to arrive (ticket per tile, left at zero) adds them in split order, converts and stores.  Used for all
    // tiles when they are few (small token counts), and for the tiles of an incomplete last wave otherwise.
    int n_whole;
    int ksplit;
    float* part;          // [split tiles][ksplit][BM*MT][BN] f32
    unsigned* counters;   // [split tiles]
    int* status;  // 0 = ok; otherwise code<<16 | detail of the first wait that expired
    long long* dbg;  // optional timeline buffer (diagnostic), CTA 0 only
    int tma_store;   // 1: whole dense tiles leave through shared memory and TMA stores (tmap_y)
};

// K-major, 128B-swizzled operand: 8-row groups are 1024 B apart (SBO), LBO unused, descriptor version 1.
__device__ __forceinline__ uint64_t umma_desc(uint32_t saddr) {
    uint64_t d = (uint64_t)((saddr & 0x3FFFFu) >> 4);
    d |= (uint64_t)1 << 16;
    d |= (uint64_t)(1024 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}

__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc, uint32_t accum) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(da), "l"(db), "r"(idesc), "r"(accum)
        : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&v)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
        "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
          "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]),
          "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]),
          "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
        : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ uint32_t hmul2u(uint32_t a, uint32_t b) {
    uint32_t r;
    asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
    return r;
}
template <int GROUP, int MT>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_w4a16_tc_kernel(const __grid_constant__ CUtensorMap tmap_x, const __grid_constant__ CUtensorMap tmap_y,
                     const GemmArgs a) {
    constexpr int NT = Cfg<MT>::NT;
    constexpr int NB = Cfg<MT>::NB;
    constexpr int A_STAGE = Cfg<MT>::A_STAGE;
    constexpr int TMEM_COLS = Cfg<MT>::TMEM_COLS;
    constexpr int BMT = BM * MT;
    extern __shared__ unsigned char smem_dyn[];
    __shared__ uint32_t s_tmem_base;
    __shared__ int s_abort;
    __shared__ int s_last;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t base = (smem_u32(smem_dyn) + 1023u) & ~1023u;
    unsigned char* base_ptr = smem_dyn + (base - smem_u32(smem_dyn));
    // [A ring NT x MT*16K][B ring NB x 32K][raw ring NT x 8K][barriers]; A and B bases are 1024-byte aligned
    auto a_addr = [&](int s) { return base + (uint32_t)s * A_STAGE; };
    auto b_addr = [&](int s) { return base + (uint32_t)(NT * A_STAGE) + (uint32_t)s * B_BYTES; };
    auto raw_addr = [&](int s) { return base + (uint32_t)(NT * A_STAGE + NB * B_BYTES) + (uint32_t)s * RAW_BYTES; };
    const uint32_t bars = base + NT * (A_STAGE + RAW_BYTES) + NB * B_BYTES;
    auto full_bar = [&](int s) { return bars + 8u * s; };               // TMA landed (A + raw)
    auto empty_bar = [&](int s) { return bars + 8u * (NT + s); };       // MMAs that read A[s] retired
    auto bready_bar = [&](int s) { return bars + 8u * (2 * NT + s); };  // B[s] expanded
    auto bfree_bar = [&](int s) { return bars + 8u * (2 * NT + NB + s); };  // MMAs that read B[s] retired
    const uint32_t accum_bar = bars + 8u * (2 * NT + 2 * NB);

    // tile of this CTA (groups of GROUP_M m-tiles walk the n-tiles together)
    int m0, n0, rb0, rows_valid;
    // whole tiles first, then the split ones: their CTAs run last and fill the wave the whole tiles leave incomplete
    const bool is_split = (int)blockIdx.x >= a.n_whole && a.ksplit > 1;
    const int ks = is_split ? a.ksplit : 1;
    const int sidx = is_split ? ((int)blockIdx.x - a.n_whole) / ks : 0;     // index among the split tiles
    const int split = is_split ? ((int)blockIdx.x - a.n_whole) % ks : 0;
    const int tile_id = is_split ? a.n_whole + sidx : (int)blockIdx.x;
    if (a.grouped) {
        // consecutive CTAs walk the m-tiles of one n-tile: neighbours share an expert's weight tile in L2
        const int mt = tile_id % a.m_tiles, n_tile = tile_id / a.m_tiles;
        if (mt >= *a.num_tiles) {
            return;  // the table is sized for the worst case
        }
        m0 = a.tile_row0[mt];
        rows_valid = a.tile_rows[mt];
        n0 = n_tile * BN;
        rb0 = ((a.tile_expert[mt] - a.expert0) * a.n + n0) / TILE_ROWS;
    } else {
        // groups of GROUP_M m-tiles walk the n-tiles together
        const int tile = tile_id;
        const int per_group = GROUP_M * a.n_tiles;
        const int grp = tile / per_group;
        const int first_m = grp * GROUP_M;
        const int gsz = min(GROUP_M, a.m_tiles - first_m);
        const int rem = tile - grp * per_group;
        m0 = (first_m + rem % gsz) * BMT;
        n0 = (rem / gsz) * BN;
        rb0 = n0 / TILE_ROWS;
        rows_valid = min(BMT, a.m - m0);
    }
    const int nkb_all = a.k / BK;
    const int kb0 = (int)((long long)nkb_all * split / ks);                 // this split's k-blocks: [kb0, kb0 + nkb)
    const int nkb = (int)((long long)nkb_all * (split + 1) / ks) - kb0;
    const int nrbv = min(BN, a.n - n0) / TILE_ROWS;  // valid 16-row blocks in this tile
    // 128-token blocks of this tile that hold rows: an empty second block is neither fetched nor multiplied
    const int mt_live = (MT == 2 && rows_valid <= BM) ? 1 : MT;

    const bool stamp = a.dbg != nullptr && blockIdx.x == 0;
    if (stamp && threadIdx.x == 0) {
        a.dbg[4000] = clock64();
    }
    if (threadIdx.x == 0) {
        s_abort = 0;
        for (int s = 0; s < NT; ++s) {
            mbar_init(full_bar(s), 1);
            mbar_init(empty_bar(s), 1);
        }
        for (int s = 0; s < NB; ++s) {
            mbar_init(bready_bar(s), NUM_DQ_WARPS);
            mbar_init(bfree_bar(s), 1);
        }
        mbar_init(accum_bar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&s_tmem_base)),
                     "r"(TMEM_COLS)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = s_tmem_base;
    volatile int* abort_flag = &s_abort;

    if (warp == 0) {
        // ------------------------------------------------------------------ producer
        if (lane == 0) {
            for (int it = 0; it < nkb; ++it) {
                const int s = it % NT, r = it / NT;
                if (!mbar_wait(empty_bar(s), (r & 1) ^ 1, abort_flag, a.status, (1 << 16) | it)) {
                    break;
                }
                if (stamp && it < 1000) {
                    a.dbg[it] = clock64();
                }
                mbar_expect_tx(full_bar(s), mt_live * A_BYTES + nrbv * (TILE_WORDS * 4));
#pragma unroll
                for (int mt = 0; mt < MT; ++mt) {
                    if (mt < mt_live) {
                        tma_load_2d(a_addr(s) + mt * A_BYTES, &tmap_x, (kb0 + it) * BK, m0 + mt * BM, full_bar(s));
                    }
                }
                // the tile's row blocks are contiguous at one k-block (k-block-major layout): one copy
                bulk_load(raw_addr(s), a.qt + ((size_t)(kb0 + it) * a.nrb_w + rb0) * TILE_WORDS,
                          nrbv * (TILE_WORDS * 4), full_bar(s));
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            constexpr uint32_t IDESC = (1u << 4) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
            bool ok = true;
            for (int it = 0; it < nkb && ok; ++it) {
                const int s = it % NT, r = it / NT, sb = it % NB, rb_ = it / NB;
                ok = mbar_wait(full_bar(s), r & 1, abort_flag, a.status, (2 << 16) | it) &&
                     mbar_wait(bready_bar(sb), rb_ & 1, abort_flag, a.status, (3 << 16) | it);
                if (!ok) {
                    break;
                }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                if (stamp && it < 1000) {
                    a.dbg[3000 + it] = clock64();
                }
                const uint64_t db = umma_desc(b_addr(sb));
#pragma unroll
                for (int mt = 0; mt < MT; ++mt) {
                    if (mt < mt_live) {
                        const uint64_t da = umma_desc(a_addr(s) + mt * A_BYTES);
#pragma unroll
                        for (int j = 0; j < BK / 16; ++j) {
                            umma_f16(tmem + mt * 256, da + 2 * j, db + 2 * j, IDESC, (it > 0 || j > 0) ? 1u : 0u);
                        }
                    }
                }
                umma_commit(empty_bar(s));
                umma_commit(bfree_bar(sb));
            }
            if (ok) {
                umma_commit(accum_bar);
            }
        }
        __syncwarp();
    } else {
        // ------------------------------------------------------------------ dequantise, then epilogue
        const int dw = warp - 2;
        // bank-conflict-free assignment of the 32 (g,t) slots of a tile to lanes (reads and writes)
        const int ph = lane >> 3, jj = lane & 7;
        const int t = jj & 3, g = 2 * ((t + ph) & 3) + (jj >> 2);
        const int ng = a.k / GROUP;
        bool ok = true;
        // scales of k-block `it` for this lane's two row blocks, fetched one k-block ahead
        auto load_scales = [&](int it, uint32_t (&sc)[2]) {
            sc[0] = sc[1] = 0;
            if (dw < nrbv && it < nkb) {
                const int kbi = kb0 + it;
                const uint32_t* sp = a.st + ((size_t)(rb0 + dw) * ng) * 8 + g;
                if (GROUP >= BK) {
                    sc[0] = sc[1] = __ldg(sp + (size_t)(kbi * BK / GROUP) * 8);
                } else {
                    sc[0] = __ldg(sp + (size_t)(kbi * 2) * 8);
                    sc[1] = __ldg(sp + (size_t)(kbi * 2 + 1) * 8);
                }
            }
        };
        uint32_t sc[2], sc_next[2];
        load_scales(0, sc_next);
        for (int it = 0; it < nkb && ok; ++it) {
            const int s = it % NT, r = it / NT, sb = it % NB, rb_ = it / NB;
            sc[0] = sc_next[0];
            sc[1] = sc_next[1];
            load_scales(it + 1, sc_next);
            ok = mbar_wait(full_bar(s), r & 1, abort_flag, a.status, (4 << 16) | it) &&
                 mbar_wait(bfree_bar(sb), (rb_ & 1) ^ 1, abort_flag, a.status, (6 << 16) | it);
            if (!ok) {
                break;
            }
            if (stamp && threadIdx.x == 64 && it < 1000) {
                a.dbg[1000 + it] = clock64();
            }
            {
                const int rbi = dw;
                if (rbi < nrbv) {
                    const uint4 raw = *reinterpret_cast<const uint4*>(
                        base_ptr + (raw_addr(s) - base) + rbi * (TILE_WORDS * 4) + (4 * g + t) * 16);
                    const uint32_t rw[4] = {raw.x, raw.y, raw.z, raw.w};
                    const uint32_t row_off = b_addr(sb) + (uint32_t)(rbi * TILE_ROWS + g) * 128u;
#pragma unroll
                    for (int p = 0; p < 2; ++p) {
                        uint32_t f0[4], f1[4];
                        dequant_word(rw[2 * p], f0);
                        dequant_word(rw[2 * p + 1], f1);
                        const uint32_t s2 = sc[p];
                        const uint32_t s_r0 = __byte_perm(s2, s2, 0x1010);  // (s[r0], s[r0])
                        const uint32_t s_r1 = __byte_perm(s2, s2, 0x3232);  // (s[r1], s[r1])
                        const uint32_t chunk = (uint32_t)(((4 * p + t) ^ g) << 4);
                        *reinterpret_cast<uint4*>(base_ptr + (row_off - base) + chunk) =
                            make_uint4(hmul2u(f0[0], s_r0), hmul2u(f0[2], s_r0), hmul2u(f1[0], s_r0), hmul2u(f1[2], s_r0));
                        *reinterpret_cast<uint4*>(base_ptr + (row_off - base) + 8u * 128u + chunk) =
                            make_uint4(hmul2u(f0[1], s_r1), hmul2u(f0[3], s_r1), hmul2u(f1[1], s_r1), hmul2u(f1[3], s_r1));
                    }
                }
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(bready_bar(sb));
            }
            if (stamp && threadIdx.x == 64 && it < 1000) {
                a.dbg[2000 + it] = clock64();
            }
        }
        {
            // epilogue by all 16 warps: a warp may touch TMEM lanes 32*(warp%4) .. +31; the four warps of a
            // lane quadrant take every fourth 32-column chunk
            if (ok) {
                ok = mbar_wait(accum_bar, 0, abort_flag, a.status, (5 << 16));
            }
            ok = __all_sync(0xffffffffu, ok);
            if (stamp && threadIdx.x == 64) {
                a.dbg[4001] = clock64();
            }
            if (ok) {
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const int quad = warp & 3;
                const int ncols = min(BN, a.n - n0);
                int n_staged = 0;
                for (int mc = 0; mc < mt_live * (BN / 32); ++mc) {
                    const int mt = mc / (BN / 32), c0 = (mc % (BN / 32)) * 32;
                    if (c0 >= ncols || (mc & 3) != (dw >> 2)) {
                        continue;
                    }
                    const int row_l = mt * BM + quad * 32 + lane;
                    const int row = m0 + row_l;
                    const float rw = (a.row_w != nullptr && row_l < rows_valid) ? a.row_w[row] : 1.0f;
                    // TMA-store path: every box of a dense tile (the tensor map clips at the batch's end); of a grouped
                    // tile only the boxes whose 32 rows all belong to the tile's expert segment
                    const bool staged_box = a.tma_store && ks == 1 && (!a.grouped || mt * BM + quad * 32 + 32 <= rows_valid);
                    uint32_t v[32];
                    tmem_ld32(tmem + ((uint32_t)(quad * 32) << 16) + (uint32_t)(mt * 256 + c0), v);
                    if (ks > 1) {
                        // split-K: the f32 sums of this split go to scratch as they are
                        if (row_l < rows_valid) {
                            float4* pp = reinterpret_cast<float4*>(
                                a.part + ((size_t)sidx * ks + split) * (size_t)(BMT * BN) + (size_t)row_l * BN + c0);
#pragma unroll
                            for (int i = 0; i < 32; i += 4) {
                                if (c0 + i < ncols) {
                                    pp[i / 4] = make_float4(__uint_as_float(v[i]), __uint_as_float(v[i + 1]),
                                                            __uint_as_float(v[i + 2]), __uint_as_float(v[i + 3]));
                                }
                            }
                        }
                    } else if (a.glu && staged_box) {
                        // as below, through a staging tile of 32 rows x 16 outputs (32-byte rows, no swizzle)
                        uint32_t pk[8];
#pragma unroll
                        for (int i = 0; i < 16; i += 2) {
                            const __half h0 = silu_mul_f16(__uint_as_float(v[i]) * a.out_mul, __uint_as_float(v[16 + i]) * a.out_mul);
                            const __half h1 = silu_mul_f16(__uint_as_float(v[i + 1]) * a.out_mul, __uint_as_float(v[17 + i]) * a.out_mul);
                            pk[i / 2] = (uint32_t)__half_as_ushort(h0) | ((uint32_t)__half_as_ushort(h1) << 16);
                        }
                        if (n_staged >= 2) {
                            if (lane == 0) {
                                bulk_wait_group_read<1>();
                            }
                            __syncwarp();
                        }
                        const uint32_t sbuf = base + (uint32_t)dw * 8192u + (uint32_t)(n_staged & 1) * 4096u;
                        sts128(sbuf + (uint32_t)lane * 32u, make_uint4(pk[0], pk[1], pk[2], pk[3]));
                        sts128(sbuf + (uint32_t)lane * 32u + 16u, make_uint4(pk[4], pk[5], pk[6], pk[7]));
                        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                        __syncwarp();
                        if (lane == 0) {
                            tma_store_2d(&tmap_y, sbuf, (n0 + c0) / 2, m0 + mt * BM + quad * 32);
                            bulk_commit_group();
                        }
                        ++n_staged;
                    } else if (a.glu) {
                        // a 32-column chunk = the gate sums and the up sums of the same 16 outputs
                        if (row_l < rows_valid && c0 < ncols) {
                            uint32_t pk[8];
#pragma unroll
                            for (int i = 0; i < 16; i += 2) {
                                const __half h0 = silu_mul_f16(__uint_as_float(v[i]) * a.out_mul, __uint_as_float(v[16 + i]) * a.out_mul);
                                const __half h1 = silu_mul_f16(__uint_as_float(v[i + 1]) * a.out_mul, __uint_as_float(v[17 + i]) * a.out_mul);
                                pk[i / 2] = (uint32_t)__half_as_ushort(h0) | ((uint32_t)__half_as_ushort(h1) << 16);
                            }
                            uint4* o = reinterpret_cast<uint4*>(reinterpret_cast<__half*>(a.out) + (size_t)row * (a.n / 2) +
                                                                (n0 + c0) / 2);
                            o[0] = make_uint4(pk[0], pk[1], pk[2], pk[3]);
                            o[1] = make_uint4(pk[4], pk[5], pk[6], pk[7]);
                        }
                    } else if (staged_box) {
                        // The warp's 32 rows x 32 columns go to a staging tile in the (now idle) operand rings, laid out
                        // with the tensor map's swizzle so that the 16-byte writes of a quarter-warp hit distinct banks,
                        // and leave as one TMA store: whole 128-byte lines instead of 32 scattered half-sectors per
                        // instruction.  Rows past the batch and columns past n are clipped by the tensor map.  Two
                        // staging tiles per warp: the store of one is read out while the next is filled.
                        if (a.out_mul != 1.0f) {
#pragma unroll
                            for (int i = 0; i < 32; ++i) {
                                v[i] = __float_as_uint(__uint_as_float(v[i]) * a.out_mul);
                            }
                        }
                        if (a.row_w != nullptr) {
#pragma unroll
                            for (int i = 0; i < 32; ++i) {
                                v[i] = __float_as_uint(mul_row_w(__uint_as_float(v[i]), rw));
                            }
                        }
                        if (n_staged >= 2) {
                            if (lane == 0) {
                                bulk_wait_group_read<1>();
                            }
                            __syncwarp();
                        }
                        const uint32_t sbuf = base + (uint32_t)dw * 8192u + (uint32_t)(n_staged & 1) * 4096u;
                        if (a.out_f16) {
                            const uint32_t rowp = sbuf + (uint32_t)lane * 64u, sw = (uint32_t)(lane >> 1) & 3u;
#pragma unroll
                            for (int c = 0; c < 4; ++c) {
                                uint4 pk;
                                __half2 h;
                                h = __floats2half2_rn(__uint_as_float(v[8 * c]), __uint_as_float(v[8 * c + 1]));
                                pk.x = *reinterpret_cast<uint32_t*>(&h);
                                h = __floats2half2_rn(__uint_as_float(v[8 * c + 2]), __uint_as_float(v[8 * c + 3]));
                                pk.y = *reinterpret_cast<uint32_t*>(&h);
                                h = __floats2half2_rn(__uint_as_float(v[8 * c + 4]), __uint_as_float(v[8 * c + 5]));
                                pk.z = *reinterpret_cast<uint32_t*>(&h);
                                h = __floats2half2_rn(__uint_as_float(v[8 * c + 6]), __uint_as_float(v[8 * c + 7]));
                                pk.w = *reinterpret_cast<uint32_t*>(&h);
                                sts128(rowp + (((uint32_t)c ^ sw) << 4), pk);
                            }
                        } else {
                            const uint32_t rowp = sbuf + (uint32_t)lane * 128u, sw = (uint32_t)lane & 7u;
#pragma unroll
                            for (int c = 0; c < 8; ++c) {
                                sts128(rowp + (((uint32_t)c ^ sw) << 4), make_uint4(v[4 * c], v[4 * c + 1], v[4 * c + 2], v[4 * c + 3]));
                            }
                        }
                        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                        __syncwarp();
                        if (lane == 0) {
                            if (m0 + mt * BM + quad * 32 < a.m) {   // a box wholly past the batch is not issued at all
                                tma_store_2d(&tmap_y, sbuf, n0 + c0, m0 + mt * BM + quad * 32);
                            }
                            bulk_commit_group();
                        }
                        ++n_staged;
                    } else if (row_l < rows_valid) {
                        if (a.out_mul != 1.0f) {
#pragma unroll
                            for (int i = 0; i < 32; ++i) {
                                v[i] = __float_as_uint(__uint_as_float(v[i]) * a.out_mul);
                            }
                        }
                        if (a.row_w != nullptr) {
#pragma unroll
                            for (int i = 0; i < 32; ++i) {
                                v[i] = __float_as_uint(mul_row_w(__uint_as_float(v[i]), rw));
                            }
                        }
                        if (a.out_f16) {
                            __half* o = reinterpret_cast<__half*>(a.out) + (size_t)row * a.n + n0 + c0;
#pragma unroll
                            for (int i = 0; i < 32; i += 8) {
                                if (c0 + i < ncols) {
                                    uint4 pk;
                                    __half2 h;
                                    h = __floats2half2_rn(__uint_as_float(v[i]), __uint_as_float(v[i + 1]));
                                    pk.x = *reinterpret_cast<uint32_t*>(&h);
                                    h = __floats2half2_rn(__uint_as_float(v[i + 2]), __uint_as_float(v[i + 3]));
                                    pk.y = *reinterpret_cast<uint32_t*>(&h);
                                    h = __floats2half2_rn(__uint_as_float(v[i + 4]), __uint_as_float(v[i + 5]));
                                    pk.z = *reinterpret_cast<uint32_t*>(&h);
                                    h = __floats2half2_rn(__uint_as_float(v[i + 6]), __uint_as_float(v[i + 7]));
                                    pk.w = *reinterpret_cast<uint32_t*>(&h);
                                    *reinterpret_cast<uint4*>(o + i) = pk;
                                }
                            }
                        } else {
                            float* o = reinterpret_cast<float*>(a.out) + (size_t)row * a.n + n0 + c0;
#pragma unroll
                            for (int i = 0; i < 32; i += 4) {
                                if (c0 + i < ncols) {
                                    *reinterpret_cast<uint4*>(o + i) = make_uint4(v[i], v[i + 1], v[i + 2], v[i + 3]);
                                }
                            }
                        }
                    }
                }
                if (n_staged > 0) {
                    // the staging tiles must stay in place until the TMA stores have read them
                    if (lane == 0) {
                        bulk_wait_group_read<0>();
                    }
                    __syncwarp();
                }
            }
        }
    }

    if (stamp && threadIdx.x == 64) {
        a.dbg[4002] = clock64();
    }
    if (ks > 1) {
        __threadfence();   // this thread's partial sums, before the ticket below
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TMEM_COLS) : "memory");
    }
    if (ks > 1) {
        // Every split of the tile adds a slice of its rows over all partial tiles, in split order (the same bits whatever
        // the arrival order), converts and stores.  One CTA adding all of them would read ksplit x 256 KB alone and take
        // longer than the wave it saves.  The splits of a tile are consecutive CTAs of the launch's last wave (their
        // number never exceeds the SM count), so they run at the same time; the wait for the siblings is bounded all
        // the same.  The ticket counts arrivals up to ksplit and departures up to 2 x ksplit, then returns to zero.
        if (threadIdx.x == 0) {
            int ready = 0;
            if (!*abort_flag) {
                atomicAdd(a.counters + sidx, 1u);
                const long long t0 = clock64();
                ready = 1;
                while (*reinterpret_cast<volatile unsigned*>(a.counters + sidx) < (unsigned)ks) {
                    if (clock64() - t0 > (1ll << 31)) {
                        atomicCAS(a.status, 0, (7 << 16) | (sidx & 0xffff));   // a sibling split never arrived
                        ready = 0;
                        break;
                    }
                }
                __threadfence();
            }
            s_last = ready;
        }
        __syncthreads();
        if (s_last) {
            const int ncols = min(BN, a.n - n0), c4n = ncols / 4;
            const float* base_p = a.part + (size_t)sidx * ks * (size_t)(BMT * BN);
            const int r_begin = (int)((long long)rows_valid * split / ks), r_end = (int)((long long)rows_valid * (split + 1) / ks);
            for (int idx = threadIdx.x; idx < (r_end - r_begin) * c4n; idx += NUM_THREADS) {
                const int row_l = r_begin + idx / c4n, c = (idx % c4n) * 4;
                float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
                const float* src = base_p + (size_t)row_l * BN + c;
                for (int sp0 = 0; sp0 < ks; sp0 += 8) {
                    float4 pv[8];
#pragma unroll
                    for (int q = 0; q < 8; ++q) {      // loads of up to eight splits in flight, then added in order
                        pv[q] = sp0 + q < ks ? __ldcg(reinterpret_cast<const float4*>(src + (size_t)(sp0 + q) * (BMT * BN)))
                                             : make_float4(0.f, 0.f, 0.f, 0.f);
                    }
#pragma unroll
                    for (int q = 0; q < 8; ++q) {
                        if (sp0 + q < ks) {
                            sum.x += pv[q].x;
                            sum.y += pv[q].y;
                            sum.z += pv[q].z;
                            sum.w += pv[q].w;
                        }
                    }
                }
                const int row = m0 + row_l;
                float o4[4] = {sum.x * a.out_mul, sum.y * a.out_mul, sum.z * a.out_mul, sum.w * a.out_mul};
                if (a.row_w != nullptr) {
                    const float rw = a.row_w[row];
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        o4[i] = mul_row_w(o4[i], rw);
                    }
                }
                if (a.out_f16) {
                    const __half2 h0 = __floats2half2_rn(o4[0], o4[1]), h1 = __floats2half2_rn(o4[2], o4[3]);
                    uint2 pk;
                    pk.x = *reinterpret_cast<const uint32_t*>(&h0);
                    pk.y = *reinterpret_cast<const uint32_t*>(&h1);
                    *reinterpret_cast<uint2*>(reinterpret_cast<__half*>(a.out) + (size_t)row * a.n + n0 + c) = pk;
                } else {
                    *reinterpret_cast<float4*>(reinterpret_cast<float*>(a.out) + (size_t)row * a.n + n0 + c) =
                        make_float4(o4[0], o4[1], o4[2], o4[3]);
                }
            }
            __syncthreads();
            if (threadIdx.x == 0) {
                if (atomicAdd(a.counters + sidx, 1u) == 2u * (unsigned)ks - 1u) {
                    a.counters[sidx] = 0;   // every split has read what it needed: ready for the next launch
                }
            }
        }
    }
}

EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult qr;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qr) == cudaSuccess &&
            qr == cudaDriverEntryPointSuccess) {
            fn = (EncodeTiledFn)p;
        }
    }
    return fn;
}

}  // namespace

cudaError_t gemm_init_device() {
    cudaError_t e;
#define W4_SET(G, MTV) \
    e = cudaFuncSetAttribute(gemm_w4a16_tc_kernel<G, MTV>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg<MTV>::SMEM); \
    if (e != cudaSuccess) return e;
    W4_SET(128, 1)
    W4_SET(128, 2)
    W4_SET(32, 1)
    W4_SET(32, 2)
#undef W4_SET
    return cudaSuccess;
}

int Dec::gemm(const Lin* l, const void* x, void* dst, int t, int out_kind, cudaStream_t st) {
    if (((uintptr_t)x & 15) != 0 || ((uintptr_t)dst & 15) != 0) {
        return fail("w4a16 gemm: x and dst must be 16-byte aligned");
    }
    EncodeTiledFn enc = encode_fn();
    if (!enc) {
        return fail("w4a16 gemm: cuTensorMapEncodeTiled is not available from the driver");
    }
    CUtensorMap map;
    const cuuint64_t dims[2] = {(cuuint64_t)l->k, (cuuint64_t)t};
    const cuuint64_t strides[1] = {(cuuint64_t)l->k * 2};
    const cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)BM};
    const cuuint32_t estr[2] = {1, 1};
    CUresult cr = enc(&map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void*>(x), dims, strides, box, estr,
                      CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                      CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (cr != CUDA_SUCCESS) {
        return fail("w4a16 gemm: cuTensorMapEncodeTiled failed (%d)", (int)cr);
    }
    // the outputs as 32 x 32 boxes for the epilogue's TMA stores (f16: 64-byte rows, f32: 128-byte rows)
    CUtensorMap map_y = map;
    const bool out16 = out_kind == W4A16_OUT_F16;
    bool tma_store = tune_gemm_tma_store != 0;
    if (tma_store) {
        const cuuint64_t ydims[2] = {(cuuint64_t)l->n, (cuuint64_t)t};
        const cuuint64_t ystrides[1] = {(cuuint64_t)l->n * (out16 ? 2 : 4)};
        const cuuint32_t ybox[2] = {32, 32};
        cr = enc(&map_y, out16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, dst, ydims, ystrides,
                 ybox, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, out16 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_128B,
                 CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (cr != CUDA_SUCCESS) {
            tma_store = false;   // a refused map is not an error: the per-lane stores take any layout
        }
    }
    GemmArgs a;
    a.qt = l->qt;
    a.st = (const uint32_t*)l->st;
    a.out = dst;
    a.m = t;
    a.n = l->n;
    a.k = l->k;
    a.out_f16 = out16;
    a.n_tiles = (l->n + BN - 1) / BN;
    // Tile shape and K split are chosen together by a small cost model (times in microseconds, fitted to measurements
    // on B200): a CTA takes 0.75 us per k-block with one 128-token block and 0.95 us with two (twice the tokens), 5 us
    // around its loop, and a split CTA another 4 + 6 us per token block for writing, awaiting and adding f32 partial
    // tiles.  Candidates per tile shape: whole tiles only; whole tiles plus a split last wave; every tile split
    // 2..16 ways (at least four k-blocks per split, partial tiles within 128 MB of scratch).
    const int nkb_all = l->k / BK;
    struct Choice {
        int mt, n_whole, ks;
        double cost;
    };
    Choice best{1, 0, 1, 1e30};
    for (int mtc = 1; mtc <= 2; ++mtc) {
        if ((tune_gemm_mt == 1 || tune_gemm_mt == 2) && mtc != tune_gemm_mt) {
            continue;
        }
        const int m_tiles = (t + BM * mtc - 1) / (BM * mtc);
        // a second, empty token block is neither fetched nor multiplied: its k-blocks cost what one block costs
        const bool half_empty = mtc == 2 && t <= BM;
        const double per_kb = (mtc == 2 && !half_empty) ? 0.95 : 0.75;
        const long long tiles = (long long)m_tiles * a.n_tiles;
        const double tile_bytes = (double)BM * mtc * BN * 4.0;
        auto cta_cost = [&](int nk, bool split) { return nk * per_kb + 5.0 + (split ? 4.0 + 6.0 * mtc : 0.0); };
        auto consider = [&](long long n_whole, int ks) {
            const long long split_tiles = tiles - n_whole;
            if (ks > 1 && (split_tiles > 4096 || split_tiles * ks * tile_bytes > 128.0 * (1 << 20))) {
                return;
            }
            const int nk_split = (nkb_all + ks - 1) / ks;
            double c = (double)((n_whole + sm_count - 1) / sm_count) * cta_cost(nkb_all, false);
            if (split_tiles > 0) {
                c += (double)((split_tiles * ks + sm_count - 1) / sm_count) * cta_cost(nk_split, ks > 1);
            }
            if (c < best.cost) {
                best = Choice{mtc, (int)n_whole, ks, c};
            }
        };
        if (tune_gemm_ksplit > 0) {
            consider(0, std::min(tune_gemm_ksplit, std::max(1, nkb_all)));
            continue;
        }
        consider(tiles, 1);
        if (tune_gemm_ksplit < 0) {
            continue;
        }
        const long long rem = tiles % sm_count;
        if (rem > 0 && tiles > sm_count) {
            for (int ks = 2; ks <= 16 && nkb_all / ks >= 4; ++ks) {
                consider(tiles - rem, ks);
            }
        }
        for (int ks = 2; ks <= 16 && nkb_all / ks >= 4; ++ks) {
            consider(0, ks);
        }
    }
    const int mt = best.mt;
    a.m_tiles = (t + BM * mt - 1) / (BM * mt);
    a.nrb_w = l->n / TILE_ROWS;
    a.grouped = 0;
    a.tile_expert = a.tile_row0 = a.tile_rows = a.num_tiles = nullptr;
    a.expert0 = 0;
    a.row_w = nullptr;
    a.out_mul = l->out_mul;
    a.glu = 0;
    a.status = gemm_status;
    a.dbg = dbg_buf;
    a.tma_store = tma_store ? 1 : 0;
    const int tiles = a.m_tiles * a.n_tiles;
    int n_whole = best.n_whole, ks = best.ks;
    if (ks <= 1) {
        ks = 1;
        n_whole = tiles;
    }
    const size_t tile_floats = (size_t)BM * mt * BN;
    a.n_whole = n_whole;
    a.ksplit = ks;
    a.part = nullptr;
    a.counters = nullptr;
    if (ks > 1) {
        if (int rc = ensure_scratch((size_t)(tiles - n_whole) * ks * tile_floats, tiles - n_whole, st)) {
            return rc;
        }
        a.part = part;
        a.counters = counters;
    }
    const int grid = n_whole + (tiles - n_whole) * ks;
    if (l->group == 128) {
        if (mt == 2) {
            gemm_w4a16_tc_kernel<128, 2><<<grid, NUM_THREADS, Cfg<2>::SMEM, st>>>(map, map_y, a);
        } else {
            gemm_w4a16_tc_kernel<128, 1><<<grid, NUM_THREADS, Cfg<1>::SMEM, st>>>(map, map_y, a);
        }
    } else {
        if (mt == 2) {
            gemm_w4a16_tc_kernel<32, 2><<<grid, NUM_THREADS, Cfg<2>::SMEM, st>>>(map, map_y, a);
        } else {
            gemm_w4a16_tc_kernel<32, 1><<<grid, NUM_THREADS, Cfg<1>::SMEM, st>>>(map, map_y, a);
        }
    }
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) {
        return cuda_fail("launch gemm", e);
    }
    last_kernel = "gemm_w4a16_tc_kernel<" + std::to_string(l->group) + "," + std::to_string(mt) + ">" +
                  (ks > 1 ? " split-K " + std::to_string(ks) + (n_whole > 0 ? " on the last wave" : "") : std::string());
    launches++;
    return 0;
}

// Grouped GEMM over expert segments: `l` stacks the local experts along n (n_per_expert rows each);
// xs holds the gathered rows (sorted by expert), the m-tile table lives on the device (moe.cu).
int Dec::gemm_grouped(const Lin* l, const void* xs, int xs_rows, void* out, int n_per_expert, const MoeBufs& b,
                      int max_tiles, int mt, const float* row_w, cudaStream_t st) {
    EncodeTiledFn enc = encode_fn();
    if (!enc) {
        return fail("w4a16 gemm: cuTensorMapEncodeTiled is not available from the driver");
    }
    CUtensorMap map;
    const cuuint64_t dims[2] = {(cuuint64_t)l->k, (cuuint64_t)xs_rows};
    const cuuint64_t strides[1] = {(cuuint64_t)l->k * 2};
    const cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)BM};
    const cuuint32_t estr[2] = {1, 1};
    CUresult cr = enc(&map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void*>(xs), dims, strides, box, estr,
                      CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                      CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (cr != CUDA_SUCCESS) {
        return fail("w4a16 gemm: cuTensorMapEncodeTiled failed (%d)", (int)cr);
    }
    GemmArgs a;
    a.qt = l->qt;
    a.st = (const uint32_t*)l->st;
    a.out = out;
    a.m = xs_rows;
    a.n = n_per_expert;
    a.k = l->k;
    a.out_f16 = 1;
    a.m_tiles = max_tiles;
    a.n_tiles = (n_per_expert + BN - 1) / BN;
    a.nrb_w = l->n / TILE_ROWS;
    a.grouped = 1;
    a.tile_expert = b.tile_expert;
    a.tile_row0 = b.tile_row0;
    a.tile_rows = b.tile_rows;
    a.num_tiles = b.n_tiles;
    a.expert0 = moe.e0;
    a.row_w = row_w;
    a.out_mul = l->out_mul;
    a.glu = l->glu_f > 0 ? 1 : 0;
    a.n_whole = a.m_tiles * ((n_per_expert + BN - 1) / BN);
    a.ksplit = 1;
    a.part = nullptr;
    a.counters = nullptr;
    a.status = gemm_status;
    a.dbg = nullptr;
    // outputs as 32-row boxes for the TMA-store epilogue: [rows][n] f16, or [rows][n/2] f16 after the fused silu(gate)*up
    CUtensorMap map_y = map;
    a.tma_store = 0;
    if (tune_gemm_tma_store != 0) {
        const int n_out = a.glu ? n_per_expert / 2 : n_per_expert;
        const cuuint64_t ydims[2] = {(cuuint64_t)n_out, (cuuint64_t)xs_rows};
        const cuuint64_t ystrides[1] = {(cuuint64_t)n_out * 2};
        const cuuint32_t ybox[2] = {(cuuint32_t)(a.glu ? 16 : 32), 32};
        cr = enc(&map_y, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, out, ydims, ystrides, ybox, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                 a.glu ? CU_TENSOR_MAP_SWIZZLE_NONE : CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                 CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        a.tma_store = cr == CUDA_SUCCESS ? 1 : 0;   // else the per-lane stores
    }
    const int grid = a.m_tiles * a.n_tiles;
    if (l->group == 128) {
        if (mt == 2) {
            gemm_w4a16_tc_kernel<128, 2><<<grid, NUM_THREADS, Cfg<2>::SMEM, st>>>(map, map_y, a);
        } else {
            gemm_w4a16_tc_kernel<128, 1><<<grid, NUM_THREADS, Cfg<1>::SMEM, st>>>(map, map_y, a);
        }
    } else {
        if (mt == 2) {
            gemm_w4a16_tc_kernel<32, 2><<<grid, NUM_THREADS, Cfg<2>::SMEM, st>>>(map, map_y, a);
        } else {
            gemm_w4a16_tc_kernel<32, 1><<<grid, NUM_THREADS, Cfg<1>::SMEM, st>>>(map, map_y, a);
        }
    }
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) {
        return cuda_fail("launch grouped gemm", e);
    }
    last_kernel = "gemm_w4a16_tc_kernel<" + std::to_string(l->group) + "," + std::to_string(mt) + "> (grouped)";
    launches++;
    return 0;
}

}  // namespace w4
