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

// ---- fused all-reduce of a row-parallel GEMV --------------------------------------------------------------
// Where this rank's own sums of a launch go: its own source slot of its own receive area.
__device__ __forceinline__ float* tp_own_area(const TpComm& tp, unsigned seq) {
    return tp.buf[tp.rank] + ((size_t)(seq & 1u) * tp.world + tp.rank) * tp.area_floats;
}
__device__ __forceinline__ void st_relaxed_sys_f32(float* p, float v) {
    asm volatile("st.relaxed.sys.global.f32 [%0], %1;" ::"l"(p), "f"(v) : "memory");
}

// The CTA that holds the local sums of rows [row0, row0+nrows) has just written them (f32, [token][row]) to its
// own area.  It PUSHES them into the same slot of every peer's receive area with plain peer stores over NVLink,
// then polls its own receive area until the word of every peer has replaced the sentinel -- bounded -- adds the
// ranks' values in rank order, writes the output and puts the sentinel back.  Every word says by itself whether
// it has arrived, so the exchange needs no flag and, above all, no system-scope fence (measured here at 5 us
// each with weight copies in flight).  Plain peer stores and local loads only, no second kernel, no NCCL call.  Two parities: a peer can
// be at most one launch ahead, and then writes the other half.
// The launch number advances when `done_target` row blocks of this launch have been exchanged.
// `seq_smem`: this launch's exchange number in shared memory (thread 0 reads it from the device counter after the
// launch's dependency wait); it is read here after the first barrier.
__device__ __forceinline__ void tp_exchange(const GemvArgs& a, const GemvSeg& sg, int rb_cta0, int nrows,
                                            const unsigned* seq_smem, volatile int* abort_flag, unsigned done_target,
                                            long long* dbg = nullptr) {
    const TpComm& tp = a.tp;
    auto stamp = [&](int j) {
        if (dbg != nullptr && threadIdx.x == 0) {
            unsigned long long ns;
            asm volatile("mov.u64 %0, %globaltimer;" : "=l"(ns));
            dbg[j] = (long long)ns;
        }
    };
    __syncthreads();
    const unsigned seq = *seq_smem;
    stamp(12);   // local sums written
    const int row0 = rb_cta0 * TILE_ROWS;
    const size_t par_base = (size_t)(seq & 1u) * tp.world * tp.area_floats;
    const float* own = tp_own_area(tp, seq);
    for (int i = threadIdx.x; i < nrows * a.m; i += blockDim.x) {
        const int tok = i / nrows, lr = i - tok * nrows;
        const size_t off = (size_t)tok * tp.max_rows + row0 + lr;
        const float v = own[off];
        for (int p = 0; p < tp.world; ++p) {
            if (p != tp.rank) {
                st_relaxed_sys_f32(tp.buf[p] + par_base + (size_t)tp.rank * tp.area_floats + off, v);
            }
        }
    }
    stamp(13);   // pushed to every peer
    float* recv = tp.buf[tp.rank] + par_base;
    for (int i = threadIdx.x; i < nrows * a.m; i += blockDim.x) {
        const int tok = i / nrows, lr = i - tok * nrows;
        const size_t off = (size_t)tok * tp.max_rows + row0 + lr;
        float pv[TP_MAX_WORLD];
        const long long t0 = clock64();
        bool all;
        do {
            // all ranks' loads in flight before the first word is looked at
#pragma unroll
            for (int p = 0; p < TP_MAX_WORLD; ++p) {
                pv[p] = p < tp.world ? ld_relaxed_sys_f32(recv + (size_t)p * tp.area_floats + off) : 0.f;
            }
            all = true;
#pragma unroll
            for (int p = 0; p < TP_MAX_WORLD; ++p) {
                all = all && (p >= tp.world || p == tp.rank || __float_as_uint(pv[p]) != 0xffffffffu);
            }
            if (!all && (*abort_flag || clock64() - t0 > tp.wait_cycles)) {
                *abort_flag = 1;
                atomicCAS(a.status, 0, (20 << 16) | (rb_cta0 & 0xffff));   // a peer never delivered this row block
                break;
            }
        } while (!all);
        float v = 0.f;
#pragma unroll
        for (int p = 0; p < TP_MAX_WORLD; ++p) {
            if (p < tp.world) {
                v += pv[p];   // rank order; the own slot holds this rank's sums
                // a word that never arrived is left alone: its sentinel is still in place, and writing it again
                // could erase the peer's late store, which would then be missing for good
                if (p != tp.rank && __float_as_uint(pv[p]) != 0xffffffffu) {
                    recv[(size_t)p * tp.area_floats + off] = __uint_as_float(0xffffffffu);
                }
            }
        }
        if (all) {
            if (a.out_f16) {
                reinterpret_cast<__half*>(sg.out)[(size_t)tok * sg.n + row0 + lr] = __float2half_rn(v);
            } else {
                reinterpret_cast<float*>(sg.out)[(size_t)tok * sg.n + row0 + lr] = v;
            }
        }
    }
    stamp(14);
    __syncthreads();
    stamp(15);   // summed and stored
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
