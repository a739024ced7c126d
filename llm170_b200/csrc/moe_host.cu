// Host side of the MoE path: configuration, expert residency, scratch, and the FFN call.
// Mirrors W4a16Dec::set_moe / upload_experts_resident_streamed / build_marlin_moe_arenas
// (crates/backend-gpu/src/rawcuda/w4a16_dec/upload.rs:795-812,1021-1235) and moe_ffn_dev_t
// (crates/backend-gpu/src/rawcuda/w4a16_dec/moe/mod.rs:263-447).
#include <cstdio>
#include <cstring>
#include <string>

#include "../../include/w4a16_b200.h"
#include "dec.h"

namespace w4 {

namespace {
constexpr int MOE_BM = 128;  // rows per m-tile of the grouped GEMM (256 when experts get enough rows)

std::string w13_name(int layer) { return "\x01moe." + std::to_string(layer) + ".w13"; }
std::string w2_name(int layer) { return "\x01moe." + std::to_string(layer) + ".w2"; }

template <class T>
cudaError_t dalloc(T** p, size_t count) {
    return cudaMalloc((void**)p, count * sizeof(T));
}
}  // namespace

// `retire`: keep the blocks until the decoder is freed (a captured graph may still name them)
void Dec::free_moe(bool retire) {
    void* ptrs[] = {mb.idx, mb.wt, mb.cnt, mb.off, mb.cursor, mb.pos_of_slot, mb.slot_of_pos, mb.tile_expert, mb.tile_row0,
                    mb.tile_rows, mb.n_tiles, mb.n_rows, mb.row_w, mb.xs, mb.c13, mb.act, mb.c2};
    for (void* p : ptrs) {
        if (p) {
            if (retire) {
                retired.push_back(p);
            } else {
                cudaFree(p);
            }
        }
    }
    mb = MoeBufs{};
}

// Grow-only scratch for t tokens; never grows while `st` is capturing.
int Dec::ensure_moe(int t, cudaStream_t st) {
    if ((size_t)t <= mb.cap_tokens) {
        return 0;
    }
    if (capturing(st)) {
        return fail("w4a16 moe: scratch too small during graph capture; run the call once before capturing");
    }
    cudaDeviceSynchronize();
    free_moe(true);
    const size_t slots = (size_t)t * moe.top_k;
    const int max_tiles = (int)((slots + 7) / 8) + (moe.e1 - moe.e0);   // worst case: 8-row segments
    cudaError_t e = cudaSuccess;
    auto ok = [&](cudaError_t r) {
        if (e == cudaSuccess) {
            e = r;
        }
    };
    ok(dalloc(&mb.idx, slots));
    ok(dalloc(&mb.wt, slots));
    ok(dalloc(&mb.cnt, (size_t)moe.n_experts));
    ok(dalloc(&mb.off, (size_t)moe.n_experts));
    ok(dalloc(&mb.cursor, (size_t)moe.n_experts));
    ok(dalloc(&mb.pos_of_slot, slots));
    ok(dalloc(&mb.slot_of_pos, slots));
    ok(dalloc(&mb.tile_expert, (size_t)max_tiles));
    ok(dalloc(&mb.tile_row0, (size_t)max_tiles));
    ok(dalloc(&mb.tile_rows, (size_t)max_tiles));
    ok(dalloc(&mb.n_tiles, 1));
    ok(dalloc(&mb.n_rows, 1));
    ok(dalloc(&mb.row_w, slots));
    ok(cudaMalloc(&mb.xs, slots * moe.hidden * 2));
    ok(cudaMalloc(&mb.c13, slots * 2 * moe.ffn * 2));
    ok(cudaMalloc(&mb.act, slots * moe.ffn * 2));
    ok(cudaMalloc(&mb.c2, slots * moe.hidden * 2));
    if (e != cudaSuccess) {
        free_moe();
        return cuda_fail("alloc moe scratch", e);
    }
    mb.cap_tokens = (size_t)t;
    mb.max_tiles = max_tiles;
    return 0;
}

int Dec::moe_ffn(int layer, const float* logits, const void* x16, void* y, int t, int out_kind, cudaStream_t st) {
    if (!moe.set) {
        return fail("w4a16 moe_ffn: set_moe was not called");
    }
    if (t < 1) {
        return fail("w4a16 moe_ffn: t=%d", t);
    }
    auto i13 = lins.find(w13_name(layer)), i2 = lins.find(w2_name(layer));
    if (i13 == lins.end() || i2 == lins.end()) {
        return fail("w4a16 moe_ffn: experts of layer %d are not resident", layer);
    }
    if (int rc = ensure_moe(t, st)) {
        return rc;
    }
    if (((uintptr_t)x16 & 15) != 0) {
        return fail("w4a16 moe_ffn: x must be 16-byte aligned");
    }
    const int ns = t * moe.top_k;
    const int n_local = moe.e1 - moe.e0;
    if ((long long)ns <= 8LL * moe.n_experts) {
        // decode-sized batches (on average at most 8 rows per expert): the op is weight streaming, so every
        // <=8-row segment of an expert runs through the GEMV kernel instead of a padded 128-row MMA tile
        // every expert with rows adds at most one partial segment to the ns / 8 full ones: the grid is sized for
        // this bound, and CTAs beyond the actual count leave at once
        const int est_tiles = ns < n_local ? ns : n_local;   // segments expected to be non-empty (split-K sizing)
        const int max_tiles = est_tiles + ns / 8;
        if (max_tiles > mb.max_tiles) {
            return fail("w4a16 moe_ffn: tile table too small");
        }
        if (ns <= 1024) {
            // routing and all dispatch tables in one launch; the first grouped GEMV fetches each row's token itself
            launches += launch_moe_route_small(logits, mb, t, moe.n_experts, moe.top_k, moe.e0, moe.e1, 8, st);
            if (int rc = gemv_grouped(&i13->second, x16, mb.act, 2 * moe.ffn, mb, max_tiles, est_tiles, nullptr, st,
                                      mb.slot_of_pos, moe.top_k, /*tables_fresh=*/true)) {
                return rc;
            }
        } else {
            launch_moe_topk(logits, mb.idx, mb.wt, t, moe.n_experts, moe.top_k, st);
            launch_moe_align(mb, ns, moe.n_experts, moe.e0, moe.e1, 8, st);
            launch_moe_gather(x16, mb, ns, moe.top_k, moe.hidden, st);
            launches += 5;
            if (int rc = gemv_grouped(&i13->second, mb.xs, mb.act, 2 * moe.ffn, mb, max_tiles, est_tiles, nullptr, st)) {
                return rc;
            }
        }
        // silu(gate)*up is applied by the first grouped matmul (interleaved gate / up rows): no activation pass
        if (int rc = gemv_grouped(&i2->second, mb.act, mb.c2, moe.hidden, mb, max_tiles, est_tiles, mb.row_w, st)) {
            return rc;
        }
    } else {
        // 256-row tiles (two accumulators per CTA) once the average expert segment fills most of one
        const int bm = ((long long)ns * 4 >= (long long)moe.n_experts * 3 * 256) ? 256 : MOE_BM;
        const int max_tiles = (ns + bm - 1) / bm + n_local;
        launch_moe_topk(logits, mb.idx, mb.wt, t, moe.n_experts, moe.top_k, st);
        launches += 5;
        launch_moe_align(mb, ns, moe.n_experts, moe.e0, moe.e1, bm, st);
        launch_moe_gather(x16, mb, ns, moe.top_k, moe.hidden, st);
        if (int rc = gemm_grouped(&i13->second, mb.xs, ns, mb.act, 2 * moe.ffn, mb, max_tiles, bm / 128, nullptr, st)) {
            return rc;
        }
        if (int rc = gemm_grouped(&i2->second, mb.act, ns, mb.c2, moe.hidden, mb, max_tiles, bm / 128, mb.row_w, st)) {
            return rc;
        }
    }
    launch_moe_combine(mb, y, t, moe.hidden, moe.top_k, out_kind == W4A16_OUT_F16, st);
    launches += 1;
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? 0 : cuda_fail("moe_ffn launch", e);
}

}  // namespace w4

using w4::Dec;

static cudaStream_t moe_stream(w4a16_dec* dec, void* stream) { return stream ? (cudaStream_t)stream : dec->d.stream; }

extern "C" {

int w4a16_set_moe(w4a16_dec* dec, int n_experts, int top_k, int moe_ffn, int hidden, int group, int expert_first,
                  int expert_count) {
    Dec& d = dec->d;
    if (n_experts < 1 || n_experts > 1024 || top_k < 1 || top_k > 32 || top_k > n_experts) {
        return d.fail("w4a16 set_moe: n_experts=%d top_k=%d unsupported (experts <= 1024, top_k <= 32)", n_experts, top_k);
    }
    if ((group != 32 && group != 64 && group != 128) || moe_ffn % 64 != 0 || hidden % 64 != 0 || moe_ffn % group != 0 ||
        hidden % group != 0) {
        return d.fail("w4a16 set_moe: ffn=%d hidden=%d group=%d violate the tile contract", moe_ffn, hidden, group);
    }
    if (expert_first < 0 || expert_count < 1 || expert_first + expert_count > n_experts) {
        return d.fail("w4a16 set_moe: local expert range [%d,+%d) outside 0..%d", expert_first, expert_count, n_experts);
    }
    cudaSetDevice(d.device);
    cudaDeviceSynchronize();
    d.free_moe();
    d.moe.set = true;
    d.moe.n_experts = n_experts;
    d.moe.top_k = top_k;
    d.moe.ffn = moe_ffn;
    d.moe.hidden = hidden;
    d.moe.group = group;
    d.moe.e0 = expert_first;
    d.moe.e1 = expert_first + expert_count;
    return 0;
}

static int upload_experts_impl(w4a16_dec* dec, int layer, const void* w13_q, const void* w13_s, const void* w2_q,
                               const void* w2_s, int scale_bf16, bool on_device) {
    Dec& d = dec->d;
    if (!d.moe.set) {
        return d.fail("w4a16 upload_experts: set_moe was not called");
    }
    const int ne = d.moe.e1 - d.moe.e0, f = d.moe.ffn, h = d.moe.hidden, g = d.moe.group;
    const int n13 = ne * 2 * f, n2 = ne * h;
    const std::string a = w4::w13_name(layer), b = w4::w2_name(layer);
    if (!w4::shape_ok(n13, h, g) || !w4::shape_ok(n2, f, g)) {
        return d.fail("w4a16 upload_experts: ffn=%d hidden=%d group=%d violate the tile contract", f, h, g);
    }
    cudaSetDevice(d.device);
    // w13 is stored with the gate and up row blocks of every expert interleaved, so that the first grouped matmul
    // applies silu(gate)*up itself (no activation pass, no [slots][2*ffn] round trip)
    const int glu_f = f / w4::TILE_ROWS;
    if (on_device) {
        cudaDeviceSynchronize();   // order after whatever produced the arrays on the legacy default stream
        if (int rc = d.upload_common(a.c_str(), w13_q, w13_s, n13, h, g, scale_bf16, glu_f)) {
            return rc;
        }
        return d.upload_common(b.c_str(), w2_q, w2_s, n2, f, g, scale_bf16, 0);
    }
    struct Fill {
        const unsigned char *q, *s;
        static void fn(void* user, int which, size_t off, void* dst, size_t len) {
            const Fill* me = (const Fill*)user;
            memcpy(dst, (which == 0 ? me->q : me->s) + off, len);
        }
    };
    Fill f13{(const unsigned char*)w13_q, (const unsigned char*)w13_s}, f2{(const unsigned char*)w2_q, (const unsigned char*)w2_s};
    if (int rc = d.upload_stream(a.c_str(), n13, h, g, scale_bf16, Fill::fn, &f13, glu_f)) {
        return rc;
    }
    return d.upload_stream(b.c_str(), n2, f, g, scale_bf16, Fill::fn, &f2, 0);
}

int w4a16_upload_experts(w4a16_dec* dec, int layer, const void* w13_q, const void* w13_s, const void* w2_q,
                         const void* w2_s, int scale_bf16) {
    return upload_experts_impl(dec, layer, w13_q, w13_s, w2_q, w2_s, scale_bf16, false);
}

int w4a16_upload_experts_dev(w4a16_dec* dec, int layer, const void* w13_q, const void* w13_s, const void* w2_q,
                             const void* w2_s, int scale_bf16) {
    return upload_experts_impl(dec, layer, w13_q, w13_s, w2_q, w2_s, scale_bf16, true);
}

int w4a16_moe_topk(w4a16_dec* dec, const float* logits_dev, int* idx_dev, float* wt_dev, int t, void* stream) {
    Dec& d = dec->d;
    if (!d.moe.set) {
        return d.fail("w4a16 moe_topk: set_moe was not called");
    }
    w4::launch_moe_topk(logits_dev, idx_dev, wt_dev, t, d.moe.n_experts, d.moe.top_k, moe_stream(dec, stream));
    d.launches++;
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? 0 : d.cuda_fail("moe_topk", e);
}

int w4a16_moe_ffn(w4a16_dec* dec, int layer, const float* router_logits_dev, const void* x16_dev, void* y_dev, int t,
                  int out_kind, void* stream) {
    return dec->d.moe_ffn(layer, router_logits_dev, x16_dev, y_dev, t, out_kind, moe_stream(dec, stream));
}

}  // extern "C"
