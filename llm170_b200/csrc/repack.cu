// Re-tiling of compressed-tensors int4 weights into the T64 device layout (see layout.cuh), its
// inverse, and the element-wise dequantiser used by the parity tests.
//
// Replaces the host repacker of the reference (crates/core/src/marlin.rs:2-67, called from
// crates/backend-gpu/src/rawcuda/w4a16_dec/upload.rs:99-179): here the original bytes are copied
// to the device once and re-tiled by a kernel, so load time is bounded by the H2D copy.
#include <cuda_fp16.h>

#include "internal.h"

namespace w4 {

namespace {

__device__ __forceinline__ uint32_t spread4(uint32_t four_nibbles) {
    // four_nibbles = e0 | e1<<4 | e2<<8 | e3<<12  ->  positions 0, 4, 2, 6
    const uint32_t e0 = four_nibbles & 0xFu, e1 = (four_nibbles >> 4) & 0xFu;
    const uint32_t e2 = (four_nibbles >> 8) & 0xFu, e3 = (four_nibbles >> 12) & 0xFu;
    return e0 | (e1 << 16) | (e2 << 8) | (e3 << 24);
}

__device__ __forceinline__ uint32_t gather4(uint32_t word) {
    // inverse of spread4 for the row-r0 positions (0,4,2,6)
    return (word & 0xFu) | (((word >> 16) & 0xFu) << 4) | (((word >> 8) & 0xFu) << 8) |
           (((word >> 24) & 0xFu) << 12);
}

struct WordCoord {
    int r0, kbase;
};

__device__ __forceinline__ WordCoord coord_of(size_t widx, int nrb) {
    const int w = (int)(widx & 3);
    const int lane = (int)((widx >> 2) & 31);
    const size_t tile = widx >> 7;
    const int rb = (int)(tile % (size_t)nrb);
    const int kb = (int)(tile / (size_t)nrb);
    const int g = lane >> 2, t = lane & 3, p = w >> 1, h = w & 1;
    WordCoord c;
    c.r0 = rb * TILE_ROWS + g;
    c.kbase = kb * TILE_K + 32 * p + 8 * t + 4 * h;
    return c;
}

// glu_f: 16-row blocks per gate (and per up) half of an expert when the tiles interleave them (layout.cuh), else 0
__global__ void repack_q_kernel(const uint32_t* __restrict__ q, uint32_t* __restrict__ qt, int n, int k, int glu_f) {
    const size_t total = (size_t)n * (size_t)(k / 8);
    const int nrb = n / TILE_ROWS, k8 = k / 8;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total;
         i += (size_t)gridDim.x * blockDim.x) {
        const WordCoord c = coord_of(i, nrb);
        const int r0 = glu_src_rb(c.r0 / TILE_ROWS, glu_f) * TILE_ROWS + c.r0 % TILE_ROWS;   // source row of this tile row
        const int sh = 4 * (c.kbase & 7);
        const uint32_t a = (q[(size_t)r0 * k8 + (c.kbase >> 3)] >> sh) & 0xFFFFu;
        const uint32_t b = (q[(size_t)(r0 + 8) * k8 + (c.kbase >> 3)] >> sh) & 0xFFFFu;
        qt[i] = spread4(a) | (spread4(b) << 4);
    }
}

// The same re-tiling for a CHUNK of source rows: q holds rows [16*rb0, 16*(rb0+nrbc)) of the boundary format; their
// tiles (one per k-block and row block, scattered over qt) are written in place.  Streamed uploads re-tile chunk by chunk.
__global__ void repack_q_rows_kernel(const uint32_t* __restrict__ q, uint32_t* __restrict__ qt, int n, int k, int rb0,
                                     int nrbc, int glu_f) {
    const size_t total = (size_t)nrbc * TILE_ROWS * (size_t)(k / 8);
    const int nrb = n / TILE_ROWS, k8 = k / 8;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total;
         i += (size_t)gridDim.x * blockDim.x) {
        const WordCoord c = coord_of(i, nrbc);          // coordinates inside the chunk (row blocks 0..nrbc-1)
        const int sh = 4 * (c.kbase & 7);
        const uint32_t a = (q[(size_t)c.r0 * k8 + (c.kbase >> 3)] >> sh) & 0xFFFFu;
        const uint32_t b = (q[(size_t)(c.r0 + 8) * k8 + (c.kbase >> 3)] >> sh) & 0xFFFFu;
        const size_t tile = i >> 7;
        const int rb = (int)(tile % (size_t)nrbc), kb = (int)(tile / (size_t)nrbc);
        qt[((size_t)kb * nrb + glu_dest_rb(rb0 + rb, glu_f)) * TILE_WORDS + (i & 127)] = spread4(a) | (spread4(b) << 4);
    }
}

__global__ void unpack_q_kernel(const uint32_t* __restrict__ qt, uint32_t* __restrict__ q, int n, int k) {
    // one thread per ORIGINAL word (8 consecutive k of one row) = two packed words (h = 0, 1)
    const size_t total = (size_t)n * (size_t)(k / 8);
    const int k8 = k / 8;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total;
         i += (size_t)gridDim.x * blockDim.x) {
        const int row = (int)(i / (size_t)k8), kw = (int)(i % (size_t)k8);
        int pos0, pos1;
        const size_t w0 = word_index(row, kw * 8, n, &pos0);
        const size_t w1 = word_index(row, kw * 8 + 4, n, &pos1);
        const uint32_t lo = gather4(qt[w0] >> (4 * (pos0 & 1)));
        const uint32_t hi = gather4(qt[w1] >> (4 * (pos1 & 1)));
        q[i] = lo | (hi << 16);
    }
}

// bf16 scale times 2^shift as f16; *bad is set when that value is not exactly representable in f16.
__device__ __forceinline__ uint16_t bf16_to_f16_exact(uint16_t b, int shift, int* bad) {
    const float f = ldexpf(__uint_as_float(((uint32_t)b) << 16), shift);
    const __half h = __float2half_rn(f);
    if (__half2float(h) != f && !(f != f)) {
        *bad = 1;
    }
    return __half_as_ushort(h);
}

// Smallest and largest biased exponent among the non-zero bf16 scales (range[0] starts at 255, range[1] at 0).
__global__ void scale_range_kernel(const uint16_t* __restrict__ s, size_t total, int* __restrict__ range) {
    int lo = 255, hi = 0;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const int v = s[i] & 0x7fff;
        if (v != 0) {
            const int e = v >> 7;
            lo = min(lo, e);
            hi = max(hi, e);
        }
    }
    lo = __reduce_min_sync(0xffffffffu, lo);
    hi = __reduce_max_sync(0xffffffffu, hi);
    if ((threadIdx.x & 31) == 0) {
        atomicMin(range, lo);
        atomicMax(range + 1, hi);
    }
}

// `ng`: groups per row of the TILED array; a source group covers `src_div` of them (2 when 64-channel groups are
// stored as two 32-channel groups with the same scale, else 1).
__global__ void repack_s_kernel(const uint16_t* __restrict__ s, uint16_t* __restrict__ stl, int n, int ng, int src_div,
                                int scale_bf16, int shift, int* __restrict__ err, int glu_f) {
    const size_t total = (size_t)n * (size_t)ng;
    const int ng_src = ng / src_div;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total;
         i += (size_t)gridDim.x * blockDim.x) {
        // i indexes the tiled array: [rb][grp][j][hi]
        const int hi = (int)(i & 1), j = (int)((i >> 1) & 7);
        const size_t rg = i >> 4;
        const int grp = (int)(rg % (size_t)ng), rb = glu_src_rb((int)(rg / (size_t)ng), glu_f);
        uint16_t v = s[(size_t)(rb * TILE_ROWS + j + 8 * hi) * ng_src + grp / src_div];
        if (scale_bf16) {
            int bad = 0;
            v = bf16_to_f16_exact(v, shift, &bad);
            if (bad && err) {
                *err = 1;
            }
        }
        stl[i] = v;
    }
}

// Scales of a chunk of source rows: the tiled array keeps a row block's groups together, so the chunk's tiles are the
// contiguous range starting at row block rb0.
__global__ void repack_s_rows_kernel(const uint16_t* __restrict__ s, uint16_t* __restrict__ stl, int ng, int src_div,
                                     int scale_bf16, int shift, int* __restrict__ err, int rb0, int nrbc, int glu_f) {
    const size_t total = (size_t)nrbc * TILE_ROWS * (size_t)ng;
    const int ng_src = ng / src_div;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total;
         i += (size_t)gridDim.x * blockDim.x) {
        const int hi = (int)(i & 1), j = (int)((i >> 1) & 7);
        const size_t rg = i >> 4;
        const int grp = (int)(rg % (size_t)ng), rb = (int)(rg / (size_t)ng);
        uint16_t v = s[(size_t)(rb * TILE_ROWS + j + 8 * hi) * ng_src + grp / src_div];
        if (scale_bf16) {
            int bad = 0;
            v = bf16_to_f16_exact(v, shift, &bad);
            if (bad && err) {
                *err = 1;
            }
        }
        stl[(size_t)glu_dest_rb(rb0 + rb, glu_f) * ng * 16 + (i - (size_t)rb * ng * 16)] = v;
    }
}

__global__ void unpack_s_kernel(const uint16_t* __restrict__ stl, uint16_t* __restrict__ s, int n, int ng, int src_div) {
    const size_t total = (size_t)n * (size_t)ng;
    const int ng_src = ng / src_div;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total;
         i += (size_t)gridDim.x * blockDim.x) {
        const int hi = (int)(i & 1), j = (int)((i >> 1) & 7);
        const size_t rg = i >> 4;
        const int grp = (int)(rg % (size_t)ng), rb = (int)(rg / (size_t)ng);
        if (grp % src_div == 0) {
            s[(size_t)(rb * TILE_ROWS + j + 8 * hi) * ng_src + grp / src_div] = stl[i];
        }
    }
}

// (nibble - 8) * scale in f32 -- exact: 4 significant bits times 11 -- for every element.
// Follows crates/core/src/matmul/cpu.rs:167-194.  OUT_F16 additionally rounds once to f16 (RNE),
// which is the value the tensor-core GEMM feeds its MMA.
template <bool OUT_F16>
__global__ void dequant_kernel(const uint32_t* __restrict__ qt, const uint16_t* __restrict__ stl,
                               void* __restrict__ out, int n, int k, int group, float out_mul) {
    const size_t total = (size_t)n * (size_t)(k / 8);
    const int nrb = n / TILE_ROWS, ng = k / group;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total;
         i += (size_t)gridDim.x * blockDim.x) {
        const WordCoord c = coord_of(i, nrb);
        const uint32_t w = qt[i];
        const int rb = c.r0 / TILE_ROWS, g = c.r0 % TILE_ROWS;
        const int grp = c.kbase / group;
        const size_t sbase = (((size_t)rb * ng + grp) * 8 + g) * 2;
        // out_mul is a power of two (1 unless the source scales were bf16 values outside the f16 range)
        const float s0 = __half2float(__ushort_as_half(stl[sbase])) * out_mul;
        const float s1 = __half2float(__ushort_as_half(stl[sbase + 1])) * out_mul;
        const int pos[4] = {0, 4, 2, 6};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const float v0 = (float)((int)((w >> (4 * pos[e])) & 0xFu) - 8) * s0;
            const float v1 = (float)((int)((w >> (4 * (pos[e] + 1))) & 0xFu) - 8) * s1;
            const size_t o0 = (size_t)c.r0 * k + c.kbase + e;
            const size_t o1 = (size_t)(c.r0 + 8) * k + c.kbase + e;
            if (OUT_F16) {
                ((__half*)out)[o0] = __float2half_rn(v0);
                ((__half*)out)[o1] = __float2half_rn(v1);
            } else {
                ((float*)out)[o0] = v0;
                ((float*)out)[o1] = v1;
            }
        }
    }
}

// Lane-order mirror of the CPU dot product, for parity gates: one warp per output element keeps the 64 f32 lane
// accumulators of crates/core/src/quant/lane.rs:42-70 (lane l owns elements i = l mod 64, in increasing i, with the
// multiply and the add rounded separately), two per thread, and combines them in f64 with the fixed tree of
// lane.rs:2-13 (i += i+32, then offsets 16, 8, 4, 2, 1).  Bit-identical to the reference's lane dot for any
// token count; it plays the role of the reference's FFMA mirror kernel w4a16_gemm_g128
// (crates/backend-gpu/src/rawcuda/assets/gptq4.cu:825-951), which its gate compares bit for bit with lane.rs.
__global__ void lane_mirror_kernel(const uint32_t* __restrict__ qt, const uint16_t* __restrict__ stl,
                                   const __half* __restrict__ x, float* __restrict__ out, int n, int k, int group,
                                   float out_mul) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int row = blockIdx.x * 8 + warp, tok = blockIdx.y;
    if (row >= n) {
        return;
    }
    const int ng = k / group;
    const int rb = row / TILE_ROWS, rr = row % TILE_ROWS;
    const uint16_t* srow = stl + ((size_t)rb * ng * 8 + (rr & 7)) * 2 + (rr >> 3);   // + grp * 16
    const __half* xr = x + (size_t)tok * k;
    float acc[2] = {0.f, 0.f};
    for (int i0 = 0; i0 < k; i0 += 64) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int i = i0 + lane + 32 * h;
            int pos;
            const size_t wi = word_index(row, i, n, &pos);
            const int nib = (int)((qt[wi] >> (4 * pos)) & 0xFu);
            const float sc = __half2float(__ushort_as_half(srow[(size_t)(i / group) * 16])) * out_mul;
            const float w = __fmul_rn((float)(nib - 8), sc);
            acc[h] = __fadd_rn(acc[h], __fmul_rn(w, __half2float(xr[i])));
        }
    }
    double a = (double)acc[0] + (double)acc[1];
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
        a += __shfl_down_sync(0xffffffffu, a, off);
    }
    if (lane == 0) {
        out[(size_t)tok * n + row] = (float)a;
    }
}

// f32 activations -> f16 (round to nearest even; exact for the f16-valued f32 the reference's norm kernels emit),
// the role of w4a16_cast_f16 (crates/backend-gpu/src/rawcuda/assets/moepp.cu:36-51)
__global__ void cast_f16_kernel(const float* __restrict__ x, __half* __restrict__ y, size_t total) {
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        y[i] = __float2half_rn(x[i]);
    }
}

inline int grid_for(size_t total) {
    size_t b = (total + 255) / 256;
    if (b > 148 * 32) {
        b = 148 * 32;
    }
    return b < 1 ? 1 : (int)b;
}

}  // namespace

void launch_repack_q(const uint32_t* q, uint32_t* qt, int n, int k, int glu_f, cudaStream_t st) {
    repack_q_kernel<<<grid_for((size_t)n * (k / 8)), 256, 0, st>>>(q, qt, n, k, glu_f);
}
void launch_lane_mirror(const uint32_t* qt, const uint16_t* stl, const void* x16, float* out, int n, int k, int group,
                        int t, float out_mul, cudaStream_t st) {
    lane_mirror_kernel<<<dim3((n + 7) / 8, t), 256, 0, st>>>(qt, stl, (const __half*)x16, out, n, k, group, out_mul);
}
void launch_cast_f16(const float* x, void* y16, size_t total, cudaStream_t st) {
    cast_f16_kernel<<<grid_for(total), 256, 0, st>>>(x, (__half*)y16, total);
}
void launch_scale_range(const uint16_t* s, size_t total, int* range2, cudaStream_t st) {
    scale_range_kernel<<<grid_for(total), 256, 0, st>>>(s, total, range2);
}
void launch_repack_s(const uint16_t* s, uint16_t* stl, int n, int k, int group, int src_div, int scale_bf16, int shift,
                     int* err, int glu_f, cudaStream_t st) {
    repack_s_kernel<<<grid_for((size_t)n * (k / group)), 256, 0, st>>>(s, stl, n, k / group, src_div, scale_bf16, shift, err,
                                                                       glu_f);
}
void launch_repack_q_rows(const uint32_t* q_chunk, uint32_t* qt, int n, int k, int rb0, int nrbc, int glu_f,
                          cudaStream_t st) {
    repack_q_rows_kernel<<<grid_for((size_t)nrbc * TILE_ROWS * (k / 8)), 256, 0, st>>>(q_chunk, qt, n, k, rb0, nrbc, glu_f);
}
void launch_repack_s_rows(const uint16_t* s_chunk, uint16_t* stl, int n, int k, int group, int src_div, int scale_bf16,
                          int shift, int* err, int rb0, int nrbc, int glu_f, cudaStream_t st) {
    (void)n;
    repack_s_rows_kernel<<<grid_for((size_t)nrbc * TILE_ROWS * (k / group)), 256, 0, st>>>(
        s_chunk, stl, k / group, src_div, scale_bf16, shift, err, rb0, nrbc, glu_f);
}
void launch_unpack_q(const uint32_t* qt, uint32_t* q, int n, int k, cudaStream_t st) {
    unpack_q_kernel<<<grid_for((size_t)n * (k / 8)), 256, 0, st>>>(qt, q, n, k);
}
void launch_unpack_s(const uint16_t* stl, uint16_t* s, int n, int k, int group, int src_div, cudaStream_t st) {
    unpack_s_kernel<<<grid_for((size_t)n * (k / group)), 256, 0, st>>>(stl, s, n, k / group, src_div);
}
void launch_dequant(const uint32_t* qt, const uint16_t* stl, void* out, int n, int k, int group, int out_f16,
                    float out_mul, cudaStream_t st) {
    const int g = grid_for((size_t)n * (k / 8));
    if (out_f16) {
        dequant_kernel<true><<<g, 256, 0, st>>>(qt, stl, out, n, k, group, out_mul);
    } else {
        dequant_kernel<false><<<g, 256, 0, st>>>(qt, stl, out, n, k, group, out_mul);
    }
}

}  // namespace w4
