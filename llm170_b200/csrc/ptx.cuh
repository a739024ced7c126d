// Thin inline-PTX helpers shared by the kernels: mbarriers with bounded waits, bulk (TMA) copies,
// and the int4 -> f16 register expansion of the T64 layout.
#pragma once
#include <cuda.h>
#include <cuda_fp16.h>

#include <cstdint>

namespace w4 {

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_init_fence() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}

// Bounded wait on an mbarrier phase. Gives up after 2^31 cycles (about a second), or as soon as another
// thread of the CTA has given up (*abort_flag, in shared memory); the first to give up records `code`
// in the global status word. Returns false if it gave up: the caller must fall through to its exit.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int* status,
                                          int code) {
    if (mbar_try(bar, parity)) {
        return true;
    }
    const long long t0 = clock64();
    unsigned spins = 0;
    while (!mbar_try(bar, parity)) {
        if ((++spins & 0x3FF) == 0) {
            if (*abort_flag) {
                return false;
            }
            if (clock64() - t0 > (1ll << 31)) {
                *abort_flag = 1;
                atomicCAS(status, 0, code);
                return false;
            }
        }
    }
    return true;
}

// 1-D bulk copy global -> shared, completion counted in bytes on an mbarrier.
// Both addresses 16-byte aligned, size a multiple of 16.
__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
                 "l"(src), "r"(bytes), "r"(bar)
                 : "memory");
}

// 2-D tiled TMA load into this CTA only. c0 = innermost coordinate (elements), c1 = row.
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int c0, int c1, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(bar)
        : "memory");
}

// 2-D tiled TMA store shared -> global (bulk async group of the issuing thread). c0 = innermost coordinate.
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, uint32_t src, int c0, int c1) {
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.tile.bulk_group [%0, {%1, %2}], [%3];" ::"l"(map), "r"(c0),
                 "r"(c1), "r"(src)
                 : "memory");
}
// 16 / 4 bytes per thread, global -> shared, without passing through registers (asynchronous copy)
__device__ __forceinline__ void cp_async_16(uint32_t dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_4(uint32_t dst, const void* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait_group() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_all;" ::: "memory"); }
__device__ __forceinline__ void bulk_commit_group() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// waits until all but the newest N bulk groups of this thread have finished READING their shared-memory source
template <int N> __device__ __forceinline__ void bulk_wait_group_read() {
    asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void sts128(uint32_t addr, uint4 v) {
    asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

__device__ __forceinline__ uint32_t lds32(uint32_t addr) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}
__device__ __forceinline__ float2 lds_f32x2(uint32_t addr) {
    float2 v;
    asm volatile("ld.shared.v2.f32 {%0,%1}, [%2];" : "=f"(v.x), "=f"(v.y) : "r"(addr));
    return v;
}

__device__ __forceinline__ uint32_t lop3_and_or(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t r;
    asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(r) : "r"(a), "r"(b), "r"(c));
    return r;
}

// Routing weight applied to a grouped-matmul output the way the reference's MoE GEMM does it
// (crates/backend-gpu/src/rawcuda/assets/marlin_moe/marlin_template.h:1515-1524): the f32 sum is rounded to f16,
// the weight is rounded to f16, and their product is rounded to f16 once more (__hmul2 there).  Returned as f32.
__device__ __forceinline__ float mul_row_w(float v, float w) {
    return __half2float(__hmul(__float2half_rn(v), __float2half_rn(w)));
}

// silu(gate) * up the way the reference's activation kernel computes it (crates/backend-gpu/src/rawcuda/assets/moe.cu:
// 1649-1660) on the f16-rounded outputs of the first grouped matmul: both sums are rounded to f16, the product is
// formed in f32 and rounded to f16 once.
__device__ __forceinline__ __half silu_mul_f16(float gate_sum, float up_sum) {
    const float g = __half2float(__float2half_rn(gate_sum)), u = __half2float(__float2half_rn(up_sum));
    return __float2half_rn((g / (1.0f + expf(-g))) * u);
}

// One packed word of the T64 layout -> a[0]=(r0;k,k+1) a[1]=(r1;k,k+1) a[2]=(r0;k+2,k+3) a[3]=(r1;k+2,k+3)
// as half2 registers holding (nibble-8) exactly.  0x6400 is f16 1024: (w & 0x000f)|0x6400 = 1024+nibble,
// minus 1032 = nibble-8;  (w & 0x00f0)|0x6400 = 1024+16*nibble, times 1/16 minus 72 = nibble-8.
__device__ __forceinline__ void dequant_word(uint32_t w, uint32_t (&a)[4]) {
    const uint32_t MAGIC = 0x64006400u, SUB = 0x64086408u, MUL = 0x2c002c00u, ADD = 0xd480d480u;
    const uint32_t w8 = w >> 8;
    const uint32_t lo0 = lop3_and_or(w, 0x000f000fu, MAGIC), hi0 = lop3_and_or(w, 0x00f000f0u, MAGIC);
    const uint32_t lo1 = lop3_and_or(w8, 0x000f000fu, MAGIC), hi1 = lop3_and_or(w8, 0x00f000f0u, MAGIC);
    asm("sub.f16x2 %0, %1, %2;" : "=r"(a[0]) : "r"(lo0), "r"(SUB));
    asm("fma.rn.f16x2 %0, %1, %2, %3;" : "=r"(a[1]) : "r"(hi0), "r"(MUL), "r"(ADD));
    asm("sub.f16x2 %0, %1, %2;" : "=r"(a[2]) : "r"(lo1), "r"(SUB));
    asm("fma.rn.f16x2 %0, %1, %2, %3;" : "=r"(a[3]) : "r"(hi1), "r"(MUL), "r"(ADD));
}

// Same word -> the raw nibbles as f16 SUBNORMALS: a[0], a[2] hold nibble * 2^-24 (rows r0) and a[1], a[3]
// hold nibble * 2^-20 (rows r1).  Exact; the caller removes the power of two and the zero point 8
// in the f32 accumulator domain.
__device__ __forceinline__ void nibbles_as_subnormals(uint32_t w, uint32_t (&a)[4]) {
    const uint32_t w8 = w >> 8;
    a[0] = w & 0x000f000fu;
    a[1] = w & 0x00f000f0u;
    a[2] = w8 & 0x000f000fu;
    a[3] = w8 & 0x00f000f0u;
}

}  // namespace w4
