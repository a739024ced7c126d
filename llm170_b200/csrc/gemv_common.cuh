// Pieces shared by the decode GEMV kernels (gemv.cu, gemv_sk.cu).
#pragma once
#include <cuda_fp16.h>

#include "internal.h"
#include "ptx.cuh"

namespace w4 {

constexpr int CTA_RB = 16;                        // 16 row blocks = 256 rows per CTA
constexpr int ROWS_PER_CTA = CTA_RB * TILE_ROWS;
constexpr int CK = 2;                             // k-blocks per ring stage
constexpr int KB_BYTES = CTA_RB * TILE_WORDS * 4; // 8 KB: one k-block of the CTA's rows
constexpr int STAGE_BYTES = CK * KB_BYTES;        // 16 KB

__device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// first MMA of a group: accumulates onto zero
__device__ __forceinline__ void mma16816_z(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%10,%10,%10,%10};"
        : "=f"(c[0]), "=f"(c[1]), "=f"(c[2]), "=f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "f"(0.f));
}

// first MMA of a group when the accumulator starts from given values (the zero-point term of the group)
__device__ __forceinline__ void mma16816_c(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1,
                                           const float4& c) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%10,%11,%12,%13};"
        : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "f"(c.x), "f"(c.y), "f"(c.z), "f"(c.w));
}

__device__ __forceinline__ void st_release_sys(unsigned* p, unsigned v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned ld_acquire_sys(const unsigned* p) {
    unsigned v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ float ld_relaxed_sys_f32(const float* p) {
    float v;
    asm volatile("ld.relaxed.sys.global.f32 %0, [%1];" : "=f"(v) : "l"(p) : "memory");
    return v;
}

__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ float ld_dsmem_f32(uint32_t local_addr, unsigned cta_rank) {
    uint32_t ra;
    float v;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(ra) : "r"(local_addr), "r"(cta_rank));
    asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(ra) : "memory");
    return v;
}

// Fused all-reduce of a row-parallel GEMV: the CTA that holds the local sums of rows [row0, row0+nrows) has
// just written them (f32) to this rank's parity buffer.  It tells every peer (one flag per rank and row
// block, written with release.sys into the PEER's flag array), waits -- bounded -- until every peer's flag for
// this row block has reached this launch's number, then adds the peers' partial rows in rank order with
// plain peer loads over NVLink and writes the final output.  No multicast, no second kernel, no NCCL call.
// Parity buffers: a peer can be at most one launch ahead, and then writes the other buffer.
// `flag_idx` numbers the row block within the launch (the same on every rank); the launch number advances when
// `done_target` row blocks of this launch have been exchanged.
__device__ __forceinline__ void tp_exchange(const GemvArgs& a, const GemvSeg& sg, int rb_cta0, int nrows, unsigned seq,
                                            volatile int* abort_flag, int flag_idx, unsigned done_target) {
    const TpComm& tp = a.tp;
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence_system();
        for (int p = 0; p < tp.world; ++p) {
            if (p != tp.rank) {
                st_release_sys(tp.flags[p] + tp.rank * TP_MAX_CTAS + flag_idx, seq);
            }
        }
    }
    if ((int)threadIdx.x < tp.world && (int)threadIdx.x != tp.rank) {
        const unsigned* f = tp.flags[tp.rank] + threadIdx.x * TP_MAX_CTAS + flag_idx;
        const long long t0 = clock64();
        while ((int)(ld_acquire_sys(f) - seq) < 0) {
            if (*abort_flag || clock64() - t0 > (1ll << 31)) {
                *abort_flag = 1;
                atomicCAS(a.status, 0, (20 << 16) | (int)threadIdx.x);   // peer never arrived
                break;
            }
        }
    }
    __syncthreads();
    if (!*abort_flag) {
        const size_t par = (size_t)(seq & 1u) * tp.area_floats;
        const int row0 = rb_cta0 * TILE_ROWS;
        for (int i = threadIdx.x; i < nrows * a.m; i += blockDim.x) {
            const int lr = i % nrows, tok = i / nrows;
            const size_t off = par + (size_t)(row0 + lr) * GEMV_MAX_M + tok;
            float v = 0.f;
            for (int p = 0; p < tp.world; ++p) {
                v += ld_relaxed_sys_f32(tp.buf[p] + off);
            }
            if (a.out_f16) {
                reinterpret_cast<__half*>(sg.out)[(size_t)tok * sg.n + row0 + lr] = __float2half_rn(v);
            } else {
                reinterpret_cast<float*>(sg.out)[(size_t)tok * sg.n + row0 + lr] = v;
            }
        }
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        // the last row block of this launch to finish advances the launch number
        if (atomicAdd(tp.done, 1u) == done_target - 1u) {
            *tp.done = 0;
            *tp.seq = seq;
            __threadfence();
        }
    }
}

}  // namespace w4
