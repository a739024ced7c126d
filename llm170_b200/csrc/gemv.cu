// Decode-time W4A16 split-K GEMV for 1..8 tokens:  y[m][n] = sum_k x[m][k] * (q[n][k]-8) * s[n][k/group].
//
// Takes the place of the reference's split-K GEMV pair (crates/backend-gpu/src/rawcuda/assets/decode.cu:46-267,
// launched from crates/backend-gpu/src/rawcuda/w4a16_dec/kernels/decode.rs:23-127) and of its FFMA
// small-batch family (crates/backend-gpu/src/rawcuda/assets/gptq4.cu:44-723).  Differences by design:
//   * the 16 rows of each mma.sync m16n8k16 are WEIGHT rows and the 8 columns are tokens, so
//     m = 1..8 all use the same kernel and no MMA row is padding;
//   * the integer part (q-8) is fed to the MMA as an exact f16 and the f32 group scale is applied to
//     the f32 accumulator once per group, so a dequantised weight is never rounded to f16;
//   * split-K partials are reduced by the last CTA to arrive (atomic ticket, no spin, fixed
//     summation order), so there is no second launch and results are reproducible.
// The kernel is HBM-bound: each lane streams 16-byte pieces of the T64 layout (layout.cuh).
#include <cuda_fp16.h>

#include "internal.h"

namespace w4 {

namespace {

__device__ __forceinline__ uint4 ldg_stream(const uint4* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}

__device__ __forceinline__ uint32_t lop3_and_or(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t r;
    asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(r) : "r"(a), "r"(b), "r"(c));
    return r;
}

// One packed word -> the four half2 registers of an m16n8k16 A fragment holding (nibble-8) exactly.
// 0x6400 is f16 1024: (w & 0x000f) | 0x6400 is 1024+nibble, minus 1032 is nibble-8;
// (w & 0x00f0) | 0x6400 is 1024+16*nibble, times 1/16 minus 72 is nibble-8.  All steps are exact.
__device__ __forceinline__ void dequant_word(uint32_t w, uint32_t (&a)[4]) {
    const uint32_t MAGIC = 0x64006400u;
    const uint32_t SUB = 0x64086408u;   // half2(1032, 1032)
    const uint32_t MUL = 0x2c002c00u;   // half2(1/16, 1/16)
    const uint32_t ADD = 0xd480d480u;   // half2(-72, -72)
    const uint32_t w8 = w >> 8;
    uint32_t lo0 = lop3_and_or(w, 0x000f000fu, MAGIC);
    uint32_t hi0 = lop3_and_or(w, 0x00f000f0u, MAGIC);
    uint32_t lo1 = lop3_and_or(w8, 0x000f000fu, MAGIC);
    uint32_t hi1 = lop3_and_or(w8, 0x00f000f0u, MAGIC);
    asm("sub.f16x2 %0, %1, %2;" : "=r"(a[0]) : "r"(lo0), "r"(SUB));
    asm("fma.rn.f16x2 %0, %1, %2, %3;" : "=r"(a[1]) : "r"(hi0), "r"(MUL), "r"(ADD));
    asm("sub.f16x2 %0, %1, %2;" : "=r"(a[2]) : "r"(lo1), "r"(SUB));
    asm("fma.rn.f16x2 %0, %1, %2, %3;" : "=r"(a[3]) : "r"(hi1), "r"(MUL), "r"(ADD));
}

__device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// K range of split `s` in units of max(group, 64) input channels, ragged splits allowed.
__device__ __host__ __forceinline__ void split_range(int k, int group, int ksplit, int s, int* kb0, int* kb1) {
    const int unit_kb = group > TILE_K ? group / TILE_K : 1;  // k-blocks per unit
    const int units = k / (unit_kb * TILE_K);
    const int u0 = (int)(((long long)units * s) / ksplit);
    const int u1 = (int)(((long long)units * (s + 1)) / ksplit);
    *kb0 = u0 * unit_kb;
    *kb1 = u1 * unit_kb;
}

__device__ __host__ __forceinline__ int max_split_kblocks(int k, int group, int ksplit) {
    int mx = 0;
    for (int s = 0; s < ksplit; ++s) {
        int a, b;
        split_range(k, group, ksplit, s, &a, &b);
        mx = (b - a) > mx ? (b - a) : mx;
    }
    return mx;
}

template <int GROUP>
__global__ void __launch_bounds__(GEMV_WARPS * 32)
gemv_w4a16_kernel(const GemvArgs a, const int x_stride /* halves per token row in smem */) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    __half* xs = reinterpret_cast<__half*>(smem_raw);
    __shared__ int s_is_last;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int split = blockIdx.y;
    const int nkb = a.k / TILE_K;
    constexpr int KB_PER_GROUP = GROUP / TILE_K > 0 ? GROUP / TILE_K : 1;   // 2 for g128, 1 for g32
    constexpr int GROUPS_PER_KB = TILE_K / GROUP > 0 ? TILE_K / GROUP : 1;  // 1 for g128, 2 for g32

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
    const int nrb = sg.n / TILE_ROWS;
    const bool warp_active = rb < nrb;

    int kb0, kb1;
    split_range(a.k, GROUP, a.ksplit, split, &kb0, &kb1);

    // stage this split's slice of x for all tokens: xs[tok][kk - 64*kb0], row stride x_stride halves
    {
        const int halves = (kb1 - kb0) * TILE_K;
        const int vec_per_row = halves / 8;
        for (int i = threadIdx.x; i < a.m * vec_per_row; i += blockDim.x) {
            const int tok = i / vec_per_row, v = i % vec_per_row;
            const uint4 val = *reinterpret_cast<const uint4*>(a.x + (size_t)tok * a.k + (size_t)kb0 * TILE_K + v * 8);
            *reinterpret_cast<uint4*>(xs + (size_t)tok * x_stride + v * 8) = val;
        }
    }
    __syncthreads();

    float tot[4] = {0.f, 0.f, 0.f, 0.f};
    if (warp_active) {
        const uint4* wp = sg.qt + ((size_t)rb * nkb + kb0) * 32 + lane;
        const int ng = a.k / GROUP;
        const uint32_t* sp = sg.st + ((size_t)rb * ng + (size_t)kb0 * GROUPS_PER_KB / KB_PER_GROUP) * 8 + g;
        const bool tok_ok = g < a.m;
        const __half* xrow = xs + (size_t)g * x_stride + 8 * t;

        constexpr int DEPTH = 4;
        uint4 wbuf[DEPTH];
        const int nloc = kb1 - kb0;
#pragma unroll
        for (int i = 0; i < DEPTH; ++i) {
            if (i < nloc) {
                wbuf[i] = ldg_stream(wp + (size_t)i * 32);
            }
        }
        float acc[4] = {0.f, 0.f, 0.f, 0.f};
        uint32_t sc = 0;
        for (int base = 0; base < nloc; base += DEPTH) {
#pragma unroll
            for (int i = 0; i < DEPTH; ++i) {
                const int kb = base + i;
                if (kb < nloc) {
                    const uint4 w = wbuf[i];
                    if (kb + DEPTH < nloc) {
                        wbuf[i] = ldg_stream(wp + (size_t)(kb + DEPTH) * 32);
                    }
                    if (GROUP >= TILE_K) {
                        if (kb % KB_PER_GROUP == 0) {
                            sc = __ldg(sp + (size_t)(kb / KB_PER_GROUP) * 8);
                        }
                    }
                    uint4 x0 = make_uint4(0, 0, 0, 0), x1 = make_uint4(0, 0, 0, 0);
                    if (tok_ok) {
                        x0 = *reinterpret_cast<const uint4*>(xrow + kb * TILE_K);
                        x1 = *reinterpret_cast<const uint4*>(xrow + kb * TILE_K + 32);
                    }
                    uint32_t fr[4];
                    dequant_word(w.x, fr);
                    mma16816(acc, fr, x0.x, x0.y);
                    dequant_word(w.y, fr);
                    mma16816(acc, fr, x0.z, x0.w);
                    if (GROUP < TILE_K) {  // g32: the first 32 k of the tile are one group
                        const uint32_t s2 = __ldg(sp + (size_t)(kb * 2) * 8);
                        const float2 sf = __half22float2(*reinterpret_cast<const __half2*>(&s2));
                        tot[0] = fmaf(acc[0], sf.x, tot[0]);
                        tot[1] = fmaf(acc[1], sf.x, tot[1]);
                        tot[2] = fmaf(acc[2], sf.y, tot[2]);
                        tot[3] = fmaf(acc[3], sf.y, tot[3]);
                        acc[0] = acc[1] = acc[2] = acc[3] = 0.f;
                    }
                    dequant_word(w.z, fr);
                    mma16816(acc, fr, x1.x, x1.y);
                    dequant_word(w.w, fr);
                    mma16816(acc, fr, x1.z, x1.w);
                    if (GROUP < TILE_K) {
                        const uint32_t s2 = __ldg(sp + (size_t)(kb * 2 + 1) * 8);
                        const float2 sf = __half22float2(*reinterpret_cast<const __half2*>(&s2));
                        tot[0] = fmaf(acc[0], sf.x, tot[0]);
                        tot[1] = fmaf(acc[1], sf.x, tot[1]);
                        tot[2] = fmaf(acc[2], sf.y, tot[2]);
                        tot[3] = fmaf(acc[3], sf.y, tot[3]);
                        acc[0] = acc[1] = acc[2] = acc[3] = 0.f;
                    } else if (kb % KB_PER_GROUP == KB_PER_GROUP - 1) {
                        const float2 sf = __half22float2(*reinterpret_cast<const __half2*>(&sc));
                        tot[0] = fmaf(acc[0], sf.x, tot[0]);
                        tot[1] = fmaf(acc[1], sf.x, tot[1]);
                        tot[2] = fmaf(acc[2], sf.y, tot[2]);
                        tot[3] = fmaf(acc[3], sf.y, tot[3]);
                        acc[0] = acc[1] = acc[2] = acc[3] = 0.f;
                    }
                }
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
    constexpr int ROWS_PER_CTA = GEMV_WARPS * TILE_ROWS;
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
    for (int i = threadIdx.x; i < ROWS_PER_CTA * a.m; i += blockDim.x) {
        const int lr = i % ROWS_PER_CTA, tok = i / ROWS_PER_CTA;
        const int row = ((int)blockIdx.x - sg.cta0) * ROWS_PER_CTA + lr;
        if (row < sg.n) {
            float sum = 0.f;
            for (int s = 0; s < a.ksplit; ++s) {
                sum += __ldcg(a.part + ((size_t)s * gridDim.x + blockIdx.x) * (ROWS_PER_CTA * GEMV_MAX_M) +
                              lr * GEMV_MAX_M + tok);
            }
            if (a.out_f16) {
                reinterpret_cast<__half*>(sg.out)[(size_t)tok * sg.n + row] = __float2half_rn(sum);
            } else {
                reinterpret_cast<float*>(sg.out)[(size_t)tok * sg.n + row] = sum;
            }
        }
    }
    if (threadIdx.x == 0) {
        a.counters[blockIdx.x] = 0;  // ready for the next launch (graph replay needs no memset)
    }
}

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

size_t gemv_smem_bytes(int k, int group, int m, int ksplit) {
    const int halves = max_split_kblocks(k, group, ksplit) * TILE_K;
    return (size_t)m * (size_t)(halves + 32) * 2;
}

size_t gemv_part_floats(int grid_x, int ksplit) {
    return ksplit > 1 ? (size_t)ksplit * grid_x * (GEMV_WARPS * TILE_ROWS * GEMV_MAX_M) : 0;
}

// Split-K so that the grid fills the machine: about `target_ctas_per_sm` CTAs per SM in one wave,
// never more splits than scale groups, and a token slice of x that fits in 64 KB of shared memory.
// (The reference sizes its split for a 70-SM part: kernels/decode.rs:3-20.)
int gemv_pick_ksplit(int grid_x, int k, int group, int m, int sm_count, int target_ctas_per_sm) {
    const int unit = group > TILE_K ? group : TILE_K;
    const int units = k / unit;
    int ks = (sm_count * target_ctas_per_sm + grid_x - 1) / grid_x;
    if (ks > units / 2) {
        ks = units / 2;  // keep at least two units of work per split
    }
    if (ks < 1) {
        ks = 1;
    }
    while (ks < units && gemv_smem_bytes(k, group, m, ks) > 64 * 1024) {
        ++ks;
    }
    return ks;
}

cudaError_t gemv_init_device() {
    cudaError_t e = cudaFuncSetAttribute(gemv_w4a16_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024);
    if (e != cudaSuccess) {
        return e;
    }
    return cudaFuncSetAttribute(gemv_w4a16_kernel<32>, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024);
}

cudaError_t launch_gemv(const GemvArgs& a, int grid_x, cudaStream_t st) {
    const int halves = max_split_kblocks(a.k, a.group, a.ksplit) * TILE_K;
    const int x_stride = halves + 32;  // byte stride = 64 (mod 128): conflict-free 128-bit reads
    const size_t smem = (size_t)a.m * x_stride * 2;
    dim3 grid(grid_x, a.ksplit);
    if (a.group == 128) {
        gemv_w4a16_kernel<128><<<grid, GEMV_WARPS * 32, smem, st>>>(a, x_stride);
    } else {
        gemv_w4a16_kernel<32><<<grid, GEMV_WARPS * 32, smem, st>>>(a, x_stride);
    }
    return cudaGetLastError();
}

}  // namespace w4
