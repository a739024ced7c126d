// int8 lm-head: per-row quantiser and the GEMV  out[t][n] = (sum_k q[n][k] * x[t][k]) * scale[n].
//
// Takes the place of W4a16Dec::upload_head (crates/backend-gpu/src/rawcuda/w4a16_dec/upload.rs:1472-1569: host threads
// quantise the bf16 matrix) and of the FFMA kernels w4a16_gemv_i8 / w4a16_gemv_i8_t
// (crates/backend-gpu/src/rawcuda/assets/head.cu:100-225, one 64-thread block per output row, launched from
// crates/backend-gpu/src/rawcuda/w4a16_dec/kernels/gemv.rs:64-110).  The lm-head is the largest weight stream of a
// decode step after the layers (vocabulary x hidden bytes), so the kernel is built for HBM bandwidth:
//   * the quantiser runs on the device, row chunks at a time, with the reference's arithmetic (f32 absmax / 127,
//     IEEE division, round half away from zero, clamp to +-127): the stored values are bit-identical to the host recipe;
//     they are kept offset-binary (q + 128) so that one byte permute puts two of them into the mantissas of two f16;
//   * a warp owns 16 whole rows at a time (no split along K, no reduction between warps): each lane streams 16 bytes
//     of row g and of row g+8 per 64 channels, expands them to exact f16 and feeds them as the 16-row operand of
//     mma.sync m16n8k16; the tokens (up to 8 per pass) are the columns;
//   * the activations are f32 in the reference.  They are staged once per CTA as TWO f16 planes, hi = f16(x) and
//     lo = f16((x - hi) * 2^11), multiplied separately and recombined in f32: the products with the exact integer
//     weights carry x to about 2^-22 instead of the 2^-11 a single f16 plane would keep.
// No wait on another CTA anywhere in this file.
#include <cuda_fp16.h>

#include <algorithm>
#include <string>

#include "../../include/w4a16_b200.h"
#include "dec.h"
#include "gemv_common.cuh"

namespace w4 {

namespace {

constexpr int HEAD_THREADS = 512;       // 16 warps
constexpr int HEAD_TOK = 8;             // tokens per pass (columns of the MMA)
constexpr int HEAD_XPAD = 16;           // bytes added to a token's row of f16 so that quarter-warps hit distinct banks

__device__ __forceinline__ float bf16_bits_to_f32(uint16_t b) { return __uint_as_float((uint32_t)b << 16); }

// One block per row: absmax, scale, quantise.  w: bf16 [rows][k] (device staging), q: offset-binary bytes [rows][k].
__global__ void __launch_bounds__(256) head_quant_kernel(const uint16_t* __restrict__ w, uint8_t* __restrict__ q,
                                                         float* __restrict__ scale, int k) {
    __shared__ float red[8];
    __shared__ float s_scale;
    const size_t row = blockIdx.x;
    const uint16_t* wr = w + row * (size_t)k;
    float amax = 0.0f;
    for (int i = threadIdx.x; i < k; i += blockDim.x) {
        amax = fmaxf(amax, fabsf(bf16_bits_to_f32(wr[i])));
    }
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) {
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
    }
    if ((threadIdx.x & 31) == 0) {
        red[threadIdx.x >> 5] = amax;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        float m = red[0];
        for (int i = 1; i < (int)(blockDim.x >> 5); ++i) {
            m = fmaxf(m, red[i]);
        }
        const float s = m > 0.0f ? __fdiv_rn(m, 127.0f) : 1.0f;
        s_scale = s;
        scale[row] = s;
    }
    __syncthreads();
    const float s = s_scale;
    uint8_t* qr = q + row * (size_t)k;
    for (int i = threadIdx.x; i < k; i += blockDim.x) {
        float v = roundf(__fdiv_rn(bf16_bits_to_f32(wr[i]), s));   // half away from zero, as f32::round
        v = fminf(fmaxf(v, -127.0f), 127.0f);
        qr[i] = (uint8_t)((int)v + 128);
    }
}

// two offset-binary bytes of `w` (selected by `sel`) -> half2 of the exact integers q = byte - 128
__device__ __forceinline__ uint32_t ob_pair_to_half2(uint32_t w, uint32_t sel) {
    const uint32_t h = __byte_perm(w, 0x64646464u, sel);   // 0x64xx = 1024 + byte
    uint32_t r;
    asm("sub.f16x2 %0, %1, %2;" : "=r"(r) : "r"(h), "r"(0x64806480u));   // - 1152
    return r;
}

struct HeadArgs {
    const uint8_t* q;
    const float* scale;
    const float* x;     // f32 [t][k], tokens [t0, t0 + tp) of it are this pass
    float* out;         // f32 [t][n]
    int n, k, t0, tp;
};

__global__ void __launch_bounds__(HEAD_THREADS, 1) head_gemv_i8_kernel(const HeadArgs a) {
    extern __shared__ __align__(16) unsigned char hsm[];
    const int k = a.k, tp = a.tp;
    const int xrow = k * 2 + HEAD_XPAD;                 // bytes of one token's f16 row
    unsigned char* xhi = hsm;
    unsigned char* xlo = hsm + (size_t)tp * xrow;
    // stage the activations: hi = f16(x), lo = f16((x - hi) * 2^11)
    for (int i = threadIdx.x; i < tp * (k / 2); i += HEAD_THREADS) {
        const int tok = i / (k / 2), c = (i - tok * (k / 2)) * 2;
        const float2 v = *reinterpret_cast<const float2*>(a.x + (size_t)(a.t0 + tok) * k + c);
        const __half h0 = __float2half_rn(v.x), h1 = __float2half_rn(v.y);
        const __half l0 = __float2half_rn((v.x - __half2float(h0)) * 2048.0f);
        const __half l1 = __float2half_rn((v.y - __half2float(h1)) * 2048.0f);
        *reinterpret_cast<__half2*>(xhi + (size_t)tok * xrow + c * 2) = __halves2half2(h0, h1);
        *reinterpret_cast<__half2*>(xlo + (size_t)tok * xrow + c * 2) = __halves2half2(l0, l1);
    }
    __syncthreads();

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, tq = lane & 3;
    const int nrb = (a.n + 15) / 16;
    const bool tok_live = g < tp;                        // this lane's column of the MMA holds a token
    const unsigned char* xh_l = xhi + (size_t)(tok_live ? g : 0) * xrow + tq * 32;
    const unsigned char* xl_l = xlo + (size_t)(tok_live ? g : 0) * xrow + tq * 32;
    const int nsteps = k / 64;
    for (int rb = blockIdx.x * (HEAD_THREADS / 32) + warp; rb < nrb; rb += gridDim.x * (HEAD_THREADS / 32)) {
        const int r0 = min(rb * 16 + g, a.n - 1), r1 = min(rb * 16 + g + 8, a.n - 1);   // clamped: loads stay in range
        const uint4* p0 = reinterpret_cast<const uint4*>(a.q + (size_t)r0 * k) + tq;
        const uint4* p1 = reinterpret_cast<const uint4*>(a.q + (size_t)r1 * k) + tq;
        float ch[4] = {0.f, 0.f, 0.f, 0.f}, cl[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll 8
        for (int s = 0; s < nsteps; ++s) {
            // 64 channels: this lane's 16 bytes of row g and of row g+8 (the four lanes of a row cover 64 contiguous bytes)
            const uint4 w0 = __ldg(p0 + s * 4), w1 = __ldg(p1 + s * 4);
            uint4 bh0 = make_uint4(0, 0, 0, 0), bh1 = bh0, bl0 = bh0, bl1 = bh0;
            if (tok_live) {
                bh0 = *reinterpret_cast<const uint4*>(xh_l + s * 128);
                bh1 = *reinterpret_cast<const uint4*>(xh_l + s * 128 + 16);
                bl0 = *reinterpret_cast<const uint4*>(xl_l + s * 128);
                bl1 = *reinterpret_cast<const uint4*>(xl_l + s * 128 + 16);
            }
            const uint32_t ww0[4] = {w0.x, w0.y, w0.z, w0.w}, ww1[4] = {w1.x, w1.y, w1.z, w1.w};
            const uint32_t xh[8] = {bh0.x, bh0.y, bh0.z, bh0.w, bh1.x, bh1.y, bh1.z, bh1.w};
            const uint32_t xl[8] = {bl0.x, bl0.y, bl0.z, bl0.w, bl1.x, bl1.y, bl1.z, bl1.w};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                // MMA j multiplies the lane's channels 4j..4j+3: the k order inside the MMA is permuted the same way
                // for the weights and for the activations, which leaves every product in place
                uint32_t af[4];
                af[0] = ob_pair_to_half2(ww0[j], 0x4140u);
                af[1] = ob_pair_to_half2(ww1[j], 0x4140u);
                af[2] = ob_pair_to_half2(ww0[j], 0x4342u);
                af[3] = ob_pair_to_half2(ww1[j], 0x4342u);
                mma16816(ch, af, xh[2 * j], xh[2 * j + 1]);
                mma16816(cl, af, xl[2 * j], xl[2 * j + 1]);
            }
        }
        // c[0], c[1]: row g, tokens 2tq, 2tq+1;  c[2], c[3]: row g+8
        const int ra = rb * 16 + g, rbb = ra + 8;
        const float sa = ra < a.n ? a.scale[ra] : 0.f, sb = rbb < a.n ? a.scale[rbb] : 0.f;
#pragma unroll
        for (int c = 0; c < 2; ++c) {
            const int tok = 2 * tq + c;
            if (tok < tp) {
                float* o = a.out + (size_t)(a.t0 + tok) * a.n;
                if (ra < a.n) {
                    o[ra] = (ch[c] + cl[c] * (1.0f / 2048.0f)) * sa;
                }
                if (rbb < a.n) {
                    o[rbb] = (ch[2 + c] + cl[2 + c] * (1.0f / 2048.0f)) * sb;
                }
            }
        }
    }
}

}  // namespace

cudaError_t head_init_device() {
    return cudaFuncSetAttribute(head_gemv_i8_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
}

}  // namespace w4

using w4::Dec;

extern "C" {

int w4a16_upload_head(w4a16_dec* dec, const void* w_bf16_host, size_t bytes, int n, int k) {
    Dec& d = dec->d;
    if (n < 1 || k < 64 || k % 64 != 0 || w_bf16_host == nullptr || bytes < (size_t)n * k * 2) {
        return d.fail("w4a16 upload_head: shape contract n=%d k=%d (k a multiple of 64) bytes=%zu", n, k, bytes);
    }
    if ((size_t)w4::HEAD_XPAD + (size_t)k * 2 > (size_t)100 * 1024) {
        return d.fail("w4a16 upload_head: k=%d: one token's two f16 planes do not fit in shared memory", k);
    }
    cudaSetDevice(d.device);
    cudaDeviceSynchronize();
    if (d.head_q) {
        d.retired.push_back(d.head_q);      // a captured graph may still name them
        d.retired.push_back(d.head_scale);
        d.weights_bytes -= (size_t)d.head_n * d.head_k + (size_t)d.head_n * 4;
        d.head_q = nullptr;
        d.head_scale = nullptr;
        d.head_n = d.head_k = 0;
    }
    uint8_t* q = nullptr;
    float* sc = nullptr;
    uint16_t* stage = nullptr;
    const int rows_chunk = (int)std::max<size_t>(1, std::min<size_t>((size_t)n, ((size_t)32 << 20) / ((size_t)k * 2)));
    cudaError_t e = cudaMalloc(&q, (size_t)n * k);
    if (e == cudaSuccess) e = cudaMalloc(&sc, (size_t)n * 4);
    if (e == cudaSuccess) e = cudaMalloc(&stage, (size_t)rows_chunk * k * 2);
    if (e != cudaSuccess) {
        cudaFree(q);
        cudaFree(sc);
        cudaFree(stage);
        return d.cuda_fail("alloc lm-head", e);
    }
    for (int r0 = 0; r0 < n && e == cudaSuccess; r0 += rows_chunk) {
        const int rows = std::min(rows_chunk, n - r0);
        e = cudaMemcpyAsync(stage, (const unsigned char*)w_bf16_host + (size_t)r0 * k * 2, (size_t)rows * k * 2,
                            cudaMemcpyHostToDevice, d.stream);
        if (e == cudaSuccess) {
            w4::head_quant_kernel<<<rows, 256, 0, d.stream>>>(stage, q + (size_t)r0 * k, sc + r0, k);
            e = cudaGetLastError();
        }
        if (e == cudaSuccess) {
            e = cudaStreamSynchronize(d.stream);   // the staging chunk is reused
        }
    }
    cudaFree(stage);
    if (e != cudaSuccess) {
        cudaFree(q);
        cudaFree(sc);
        return d.cuda_fail("quantise lm-head", e);
    }
    d.head_q = q;
    d.head_scale = sc;
    d.head_n = n;
    d.head_k = k;
    d.weights_bytes += (size_t)n * k + (size_t)n * 4;
    return 0;
}

int w4a16_head_spec(w4a16_dec* dec, int* n, int* k) {
    Dec& d = dec->d;
    if (!d.head_q) {
        return d.fail("w4a16 head: no lm-head uploaded");
    }
    if (n) *n = d.head_n;
    if (k) *k = d.head_k;
    return 0;
}

int w4a16_head_unpack(w4a16_dec* dec, void* q_host, void* scale_host) {
    Dec& d = dec->d;
    if (!d.head_q) {
        return d.fail("w4a16 head: no lm-head uploaded");
    }
    cudaSetDevice(d.device);
    const size_t nb = (size_t)d.head_n * d.head_k;
    cudaError_t e = cudaMemcpy(q_host, d.head_q, nb, cudaMemcpyDeviceToHost);
    if (e == cudaSuccess && scale_host) {
        e = cudaMemcpy(scale_host, d.head_scale, (size_t)d.head_n * 4, cudaMemcpyDeviceToHost);
    }
    if (e != cudaSuccess) {
        return d.cuda_fail("read lm-head", e);
    }
    unsigned char* b = (unsigned char*)q_host;   // offset-binary -> two's complement
    for (size_t i = 0; i < nb; ++i) {
        b[i] ^= 0x80;
    }
    return 0;
}

int w4a16_head_forward(w4a16_dec* dec, const float* x32_dev, float* out_dev, int t, void* stream) {
    Dec& d = dec->d;
    if (!d.head_q) {
        return d.fail("w4a16 head_forward: no lm-head uploaded");
    }
    if (t < 1 || t > 16) {
        return d.fail("w4a16 head_forward: t=%d, must be 1..16", t);   // the reference's limit (assets/head.cu:159)
    }
    if (((uintptr_t)x32_dev & 7) != 0 || ((uintptr_t)out_dev & 3) != 0) {
        return d.fail("w4a16 head_forward: x must be 8-byte aligned and out 4-byte aligned");
    }
    cudaStream_t st = stream ? (cudaStream_t)stream : d.stream;
    const size_t xrow = (size_t)d.head_k * 2 + w4::HEAD_XPAD;
    const int tp_max = (int)std::min<size_t>(w4::HEAD_TOK, ((size_t)200 * 1024) / (2 * xrow));
    const int nrb = (d.head_n + 15) / 16;
    const int grid = std::min(d.sm_count, (nrb + w4::HEAD_THREADS / 32 - 1) / (w4::HEAD_THREADS / 32));
    for (int t0 = 0; t0 < t; t0 += tp_max) {
        w4::HeadArgs a;
        a.q = d.head_q;
        a.scale = d.head_scale;
        a.x = x32_dev;
        a.out = out_dev;
        a.n = d.head_n;
        a.k = d.head_k;
        a.t0 = t0;
        a.tp = std::min(tp_max, t - t0);
        w4::head_gemv_i8_kernel<<<grid, w4::HEAD_THREADS, 2 * (size_t)a.tp * xrow, st>>>(a);
        cudaError_t e = cudaGetLastError();
        if (e != cudaSuccess) {
            return d.cuda_fail("launch lm-head gemv", e);
        }
        d.launches++;
    }
    d.last_kernel = "head_gemv_i8_kernel";
    return 0;
}

}  // extern "C"
