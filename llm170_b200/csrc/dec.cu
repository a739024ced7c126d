// Host side of libw4a16_b200: the decoder object (weight residency, scratch, kernel selection) and
// the extern "C" entry points declared in include/w4a16_b200.h.
//
// Mirrors the parts of the reference's W4a16Dec that sit on the W4A16 matmul path:
// weight maps (crates/backend-gpu/src/rawcuda/w4a16_dec/mod.rs:547-556), upload + repack
// (crates/backend-gpu/src/rawcuda/w4a16_dec/upload.rs:15-179), path selection
// (crates/backend-gpu/src/rawcuda/w4a16_dec/kernels/mod.rs:121-144), split-K launch policy
// (crates/backend-gpu/src/rawcuda/w4a16_dec/kernels/decode.rs:3-127) and graph capture
// (crates/backend-gpu/src/rawcuda/ctx/graph.rs:4-85).
#include "dec.h"

#include <cstdarg>
#include <cstdio>
#include <cstring>

#include "../../include/w4a16_b200.h"

namespace {
thread_local std::string g_create_error;
}

namespace w4 {

int Dec::fail(const char* fmt, ...) {
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof(buf), fmt, ap);
    va_end(ap);
    err = buf;
    return 1;
}

int Dec::cuda_fail(const char* what, cudaError_t e) {
    return fail("w4a16: %s: %s", what, cudaGetErrorString(e));
}

bool Dec::capturing(cudaStream_t st) {
    cudaStreamCaptureStatus cs = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(st, &cs) != cudaSuccess) {
        cudaGetLastError();
        return false;
    }
    return cs != cudaStreamCaptureStatusNone;
}

// Grow-only scratch. Never grows while `st` is capturing (allocation is illegal there).
int Dec::ensure_scratch(size_t part_floats, int grid_x, cudaStream_t st) {
    if (part_floats <= part_cap && (size_t)grid_x <= counters_cap) {
        return 0;
    }
    if (capturing(st)) {
        return fail("w4a16: scratch too small during graph capture; run the call once before capturing");
    }
    cudaError_t e = cudaDeviceSynchronize();
    if (e != cudaSuccess) {
        return cuda_fail("sync before scratch growth", e);
    }
    // A graph instantiated earlier keeps the addresses of the blocks it was captured with, so a superseded
    // block is only retired here (freed with the decoder), never freed while such a graph may still replay.
    if (part_floats > part_cap) {
        if (part) {
            retired.push_back(part);
            part = nullptr;
            part_cap = 0;
        }
        e = cudaMalloc(&part, part_floats * sizeof(float));
        if (e != cudaSuccess) {
            return cuda_fail("alloc split-K scratch", e);
        }
        part_cap = part_floats;
    }
    if ((size_t)grid_x > counters_cap) {
        if (counters) {
            retired.push_back(counters);
            counters = nullptr;
            counters_cap = 0;
        }
        const size_t cap = (size_t)grid_x < 4096 ? 4096 : (size_t)grid_x;
        e = cudaMalloc(&counters, cap * sizeof(unsigned));
        if (e != cudaSuccess) {
            return cuda_fail("alloc split-K tickets", e);
        }
        cudaMemset(counters, 0, cap * sizeof(unsigned));
        counters_cap = cap;
    }
    return 0;
}

void Dec::free_lin(Lin& l) {
    if (l.qt) {
        cudaFree(l.qt);
    }
    if (l.st) {
        cudaFree(l.st);
    }
    weights_bytes -= l.bytes;
    l = Lin{};
}

int Dec::upload_common(const char* name, const void* q_dev, const void* s_dev, int n, int k, int group,
                       int scale_bf16, int glu_f) {
    // q_dev/s_dev: boundary format already on the device.  Groups of 64 channels (accepted by the reference's loader,
    // crates/core/src/w4a16.rs:225-234) are kept as two groups of 32 with the same scale: the dequantised weight
    // (nibble-8)*scale is the same number, and the kernels need no third group size.
    Lin l;
    l.n = n;
    l.k = k;
    l.group_src = group;
    l.group = group == 64 ? 32 : group;
    l.glu_f = glu_f;
    const int src_div = group == 64 ? 2 : 1;
    const size_t qb = (size_t)n * (size_t)(k / 2), sb = (size_t)n * (size_t)(k / l.group) * 2;
    cudaError_t e = cudaMalloc(&l.qt, qb);
    if (e != cudaSuccess) {
        return cuda_fail("alloc weights", e);
    }
    e = cudaMalloc(&l.st, sb);
    if (e != cudaSuccess) {
        cudaFree(l.qt);
        return cuda_fail("alloc scales", e);
    }
    // bf16 scales are stored as f16.  Every bf16 value between 2^-17 and 2^15 is an f16 value; a linear whose
    // scales leave that window is shifted into it by a power of two that the kernels take out again at the end.
    int shift = 0;
    if (scale_bf16) {
        const int preset[2] = {255, 0};
        cudaMemcpyAsync(err_flag + 1, preset, sizeof(preset), cudaMemcpyHostToDevice, stream);
        launch_scale_range((const uint16_t*)s_dev, (size_t)n * (size_t)(k / group), err_flag + 1, stream);
        int range[2] = {255, 0};
        e = cudaMemcpyAsync(range, err_flag + 1, sizeof(range), cudaMemcpyDeviceToHost, stream);
        if (e == cudaSuccess) {
            e = cudaStreamSynchronize(stream);
        }
        if (e != cudaSuccess) {
            cudaFree(l.qt);
            cudaFree(l.st);
            return cuda_fail("scale range", e);
        }
        if (range[0] <= range[1]) {
            // admissible shifts: the smallest scale stays an f16 value (2^-17 and up), and 8 times the largest one
            // -- the largest dequantised weight the tensor-core GEMM forms in f16 -- stays finite (below 2^16)
            const int lo = -17 - (range[0] - 127), hi = 12 - (range[1] - 127);
            if (lo > hi) {
                cudaFree(l.qt);
                cudaFree(l.st);
                return fail("w4a16 upload %s: bf16 scales span more than the 29 binades f16 weights can hold", name);
            }
            shift = lo > 0 ? lo : (hi < 0 ? hi : 0);
        }
    }
    l.out_mul = ldexpf(1.0f, -shift);
    cudaMemsetAsync(err_flag, 0, sizeof(int), stream);
    launch_repack_q((const uint32_t*)q_dev, l.qt, n, k, glu_f, stream);
    launch_repack_s((const uint16_t*)s_dev, l.st, n, k, l.group, src_div, scale_bf16, shift, err_flag, glu_f, stream);
    int bad = 0;
    e = cudaMemcpyAsync(&bad, err_flag, sizeof(int), cudaMemcpyDeviceToHost, stream);
    if (e == cudaSuccess) {
        e = cudaStreamSynchronize(stream);
    }
    if (e != cudaSuccess || bad) {
        cudaFree(l.qt);
        cudaFree(l.st);
        if (e != cudaSuccess) {
            return cuda_fail("repack", e);
        }
        return fail("w4a16 upload %s: a bf16 scale is not representable in f16 even after shifting", name);
    }
    l.bytes = qb + sb;
    auto it = lins.find(name);
    if (it != lins.end()) {
        free_lin(it->second);
        lins.erase(it);
    }
    weights_bytes += l.bytes;
    lins[name] = l;
    return 0;
}

// Which form of the decode GEMV serves a call, with its plan and the scratch it needs.  Shared by Dec::gemv and
// the allocation-free entry point, so that both launch the same kernel with the same plan.
int Dec::gemv_select(GemvArgs& a, bool allreduce, bool own_scratch, GemvChoice& c) {
    const int t = a.m;
    c = GemvChoice{};
    c.grid_x = gemv_plan_ctas(a);   // 256-row blocks over all segments
    a.subnormal = tune_gemv_subnormal;
    a.status = gemm_status;
    a.tp = TpComm{};
    a.grouped = 0;
    a.row_w = nullptr;
    a.nrb_w = 0;
    a.rb_no_units = tune_gemv_rowblock_units ? 0 : 1;
    if (allreduce) {
        if (tp.world < 2 || tp_peer[(tp.rank + 1) % tp.world] == nullptr) {
            return fail("w4a16 allreduce gemv: call w4a16_tp_create and w4a16_tp_connect first");
        }
        if (a.nseg != 1 || a.seg[0].n > tp_max_rows || c.grid_x > TP_MAX_CTAS) {
            return fail("w4a16 allreduce gemv: n=%d exceeds the exchange buffer (%d rows)", a.seg[0].n, tp_max_rows);
        }
        a.tp = tp;
    }
    // Up to four tokens of a g128 linear with K <= 6144 and at most 48 MB of weights: CTAs that own whole rows, no
    // scratch, no ticket (gemv_rb.cu).  At its 16 warps per SM it streams at 4 to 4.7 TB/s, the persistent form's bulk
    // copies at 6 inside its loop, and a warp of the row-block form walks its K range with four k-blocks in flight.
    // Measured on B200 (us per launch, M = 1, row-block against persistent):
    //   7168 x 5120 (18 MB) 7.0 / 10.6     5120 x 6144 (16 MB) 8.0 / 9.6      17408 x 5120 (45 MB) 12.6 / 14.9
    //   5120 x 4352 (11 MB) 6.9 /  9.0     5120 x 3072 (8 MB)  5.2 / 8.5       8704 x 5120 (22 MB)  7.3 / 11.3
    //   34816 x 5120 (89 MB) 22.9 / 22.2   5120 x 8704 (22 MB) 11.1 / 10.6     5120 x 17408 (45 MB) 19.7 / 14.1
    // Every CTA of the row-block form stages all of x, so its time grows with tokens x K (qkv 7.7 / 8.6 / 9.8 us at 1 / 2 /
    // 4 tokens, o_proj 8.9 / 9.8 / 11.1) where the (row block, K split) cluster form stays flat (9.2 / 9.3 / 9.4 and
    // 9.1 / 9.3 / 9.5): beyond 11264 token-channels the latter takes over (not for the fused all-reduce, which would lose
    // the cluster reduce; the entry point with its own scratch follows the same rule so that it returns the same bits).
    // The 16-warp variant of the row-block form (all units resident at once, x beside the weights in shared memory) has no
    // such slope -- qkv 6.4 / 6.8 / 8.2 us at 1 / 2 / 4 tokens -- and keeps every call it can take.
    const size_t w_bytes = (size_t)a.seg[0].n * a.k / 2;
    const bool rb_shape = w_bytes <= ((size_t)48 << 20) && a.k <= 6144;
    const bool rb_tokens = allreduce || !tune_gemv_cluster || (size_t)t * a.k <= 11264 || gemv_ru_fits(a, sm_count);
    const bool rb_ok = tune_gemv_rowblock && gemv_rb_fits(a);
    if (rb_ok && (tune_gemv_rowblock > 1 || (rb_shape && rb_tokens))) {
        c.form = GemvChoice::ROWBLOCK;
        c.grid_x = gemv_rb_plan(a, sm_count, c.rbw);
        a.ksplit = 1;
        snprintf(c.name, sizeof(c.name), "%s", gemv_rb_variant(a, c.grid_x, c.rbw, sm_count));
        return 0;
    }
    const bool prefer_split = rb_ok && rb_shape && !rb_tokens && tune_gemv_persistent < 2;
    c.sk = sk_make_plan(a.k, a.group, t, c.grid_x, sm_count, tune_gemv_sk_stages, tune_gemv_sk_prefetch);
    // measured on B200: the persistent form wins up to 4 tokens; at 5..8 its single-CTA sum of a row block costs
    // more than the cluster reduce of the (row block, K split) form -- except for long K (down, K = 17408: 17.6-18.6
    // against 20.9-21.4 us), where that form's K splits exceed a cluster
    if (tune_gemv_persistent && c.sk.ctas > 0 && !prefer_split && (t <= 4 || tune_gemv_persistent > 1 || a.k >= 8192)) {
        c.form = GemvChoice::PERSISTENT;
        c.part_floats = sk_part_floats(c.sk);
        c.tickets = (size_t)c.grid_x;
        a.ksplit = 1;
        snprintf(c.name, sizeof(c.name), "gemv_sk_kernel<%d,%s>", a.group, a.subnormal ? "true" : "false");
        return 0;
    }
    // with its own fixed scratch the call keeps the ticketed global reduce (that scratch is what it exists for)
    const bool cluster_ok = tune_gemv_cluster && !allreduce && !own_scratch;
    int ks = tune_gemv_ksplit > 0 ? tune_gemv_ksplit
                                  : gemv_pick_ksplit(c.grid_x, a.k, a.group, t, sm_count,
                                                     (tune_gemv_cluster && !allreduce) ? 8 : 16, tune_gemv_stages);
    const int unit = a.group > TILE_K ? a.group : TILE_K;
    if (ks > a.k / unit) {
        ks = a.k / unit;
    }
    while (gemv_smem_bytes(a.k, a.group, t, ks, tune_gemv_stages) > 112 * 1024 && ks < a.k / unit) {
        ++ks;
    }
    if (gemv_smem_bytes(a.k, a.group, t, ks, tune_gemv_stages) > 112 * 1024) {
        return fail("w4a16 gemv: k=%d too large for t=%d", a.k, t);
    }
    a.ksplit = ks;
    a.ring_stages = tune_gemv_stages;
    a.cons_warps = tune_gemv_warps;
    a.cluster = (cluster_ok && ks >= 2 && ks <= 8) ? 1 : 0;
    c.form = GemvChoice::SPLIT;
    c.part_floats = gemv_part_floats(c.grid_x, ks);
    c.tickets = (size_t)c.grid_x;
    snprintf(c.name, sizeof(c.name), "gemv_w4a16_kernel<%d,%s,%d>", a.group, a.subnormal ? "true" : "false", a.cons_warps);
    return 0;
}

int Dec::gemv_run(GemvArgs& a, const GemvChoice& c, cudaStream_t st) {
    cudaError_t e;
    switch (c.form) {
    case GemvChoice::PERSISTENT:
        e = launch_gemv_sk(a, c.sk, st);
        break;
    case GemvChoice::ROWBLOCK:
        e = launch_gemv_rb(a, c.grid_x, c.rbw, sm_count, st);
        break;
    default:
        e = launch_gemv(a, c.grid_x, st);
        break;
    }
    if (e != cudaSuccess) {
        return cuda_fail("launch gemv", e);
    }
    last_kernel = c.name;
    launches++;
    return 0;
}

int Dec::gemv(const Lin* const* ls, int nseg, const void* x, void* const* outs, int t, int out_kind,
              cudaStream_t st, bool allreduce) {
    if (t < 1 || t > GEMV_MAX_M) {
        return fail("w4a16 gemv: t=%d outside 1..%d", t, GEMV_MAX_M);
    }
    if (nseg < 1 || nseg > GEMV_MAX_SEG) {
        return fail("w4a16 gemv: %d segments outside 1..%d", nseg, GEMV_MAX_SEG);
    }
    GemvArgs a{};
    a.nseg = nseg;
    a.k = ls[0]->k;
    a.group = ls[0]->group;
    for (int i = 0; i < nseg; ++i) {
        if (ls[i]->k != a.k || ls[i]->group != a.group) {
            return fail("w4a16 gemv: segments must share k and group");
        }
        a.seg[i].qt = (const uint4*)ls[i]->qt;
        a.seg[i].st = (const uint32_t*)ls[i]->st;
        a.seg[i].out = outs[i];
        a.seg[i].n = ls[i]->n;
        a.seg[i].out_mul = ls[i]->out_mul;
    }
    a.m = t;
    a.out_f16 = out_kind == W4A16_OUT_F16;
    a.x = (const uint16_t*)x;
    if (((uintptr_t)x & 15) != 0) {
        return fail("w4a16 gemv: x must be 16-byte aligned");
    }
    for (int i = 0; i < nseg; ++i) {
        // the kernels store four f32 or four f16 at a time
        if (((uintptr_t)outs[i] & 15) != 0) {
            return fail("w4a16 gemv: output %d must be 16-byte aligned", i);
        }
    }
    GemvChoice c;
    if (int rc = gemv_select(a, allreduce, false, c)) {
        return rc;
    }
    if (int rc = ensure_scratch(c.part_floats, (int)c.tickets, st)) {
        return rc;
    }
    a.pdl = tune_pdl;
    a.dbg = dbg_buf;
    a.dbg_seq = (int)(launches % DBG_LAUNCHES);
    a.part = part;
    a.counters = counters;
    return gemv_run(a, c, st);
}

// Decode-time MoE: every <=8-row segment of an expert (device table from moe.cu) is one GEMV over that
// expert's rows of the stacked matrix `l`; xs / out hold the sorted rows.  Takes the place of the reference's
// w4a16_gemv_experts_* kernels (crates/backend-gpu/src/rawcuda/assets/gptq4.cu:317-374,
// crates/backend-gpu/src/rawcuda/w4a16_dec/moe/moe_gemv.rs:92-114).
int Dec::gemv_grouped(const Lin* l, const void* xs, void* out, int n_per_expert, const MoeBufs& b, int max_tiles,
                      int est_tiles, const float* row_w, cudaStream_t st, const int* x_slot_of_pos,
                      int x_slots_per_token, bool tables_fresh) {
    if (l->glu_f > 0 && tune_gemv_warps != 8) {
        return fail("w4a16 grouped gemv: the fused gate|up form needs gemv_warps = 8");
    }
    // eight staged token rows leave little room: with a two-stage ring the scales still fit in shared memory
    // and three CTAs share an SM (measured: 177 -> 147 us for 64 tokens of the 128-expert layer)
    const int grouped_stages = 2;
    GemvArgs a{};
    a.nseg = 1;
    a.k = l->k;
    a.group = l->group;
    a.seg[0].qt = (const uint4*)l->qt;
    a.seg[0].st = (const uint32_t*)l->st;
    a.seg[0].out = out;
    a.seg[0].n = n_per_expert;
    a.seg[0].out_mul = l->out_mul;
    a.m = GEMV_MAX_M;            // sizes the staging area; each segment brings its own row count
    a.out_f16 = 1;
    a.x = (const uint16_t*)xs;
    const int cps = gemv_plan_ctas(a);  // CTAs per segment (256 rows each)
    const int grid_x = cps * max_tiles;
    int ks = tune_gemv_ksplit > 0 ? tune_gemv_ksplit
                                  : gemv_pick_ksplit(cps * est_tiles, a.k, a.group, GEMV_MAX_M, sm_count, 8, grouped_stages);
    if (ks > 8) {
        ks = 8;  // the splits of a segment always reduce inside a cluster (no global scratch per segment)
    }
    const int unit = a.group > TILE_K ? a.group : TILE_K;
    if (ks > a.k / unit) {
        ks = a.k / unit;
    }
    if (gemv_smem_bytes(a.k, a.group, GEMV_MAX_M, ks, grouped_stages) > 112 * 1024) {
        return fail("w4a16 grouped gemv: k=%d too large", a.k);
    }
    a.ksplit = ks;
    a.subnormal = tune_gemv_subnormal;
    a.pdl = tune_pdl;
    a.glu = l->glu_f > 0 ? 1 : 0;
    a.ring_stages = grouped_stages;
    a.cons_warps = tune_gemv_warps;
    a.cluster = ks >= 2 ? 1 : 0;
    a.status = gemm_status;
    a.dbg = dbg_buf;
    a.dbg_seq = (int)(launches % DBG_LAUNCHES);
    a.grouped = 1;
    a.ctas_per_seg = cps;
    a.expert0 = moe.e0;
    a.tile_expert = b.tile_expert;
    a.tile_row0 = b.tile_row0;
    a.tile_rows = b.tile_rows;
    a.num_tiles = b.n_tiles;
    a.row_w = row_w;
    a.x_slot_of_pos = x_slot_of_pos;
    a.x_slots_per_token = x_slots_per_token;
    a.tables_fresh = tables_fresh ? 1 : 0;
    a.nrb_w = l->n / TILE_ROWS;
    a.tp = TpComm{};
    a.part = part;
    a.counters = counters;
    cudaError_t e = launch_gemv(a, grid_x, st);
    if (e != cudaSuccess) {
        return cuda_fail("launch grouped gemv", e);
    }
    last_kernel = "gemv_w4a16_kernel<" + std::to_string(a.group) + "," + (a.subnormal ? "true" : "false") + "," +
                  std::to_string(a.cons_warps) + "> (grouped)";
    launches++;
    return 0;
}

}  // namespace w4

using w4::Dec;
using w4::Lin;

static cudaStream_t pick_stream(w4a16_dec* dec, void* stream) {
    return stream ? (cudaStream_t)stream : dec->d.stream;
}

// exchange block of the fused all-reduce: header (launch counter, done counter), then the receive areas
static const size_t TP_HEADER = 4096;

extern "C" {

int w4a16_dec_new(int device, w4a16_dec** out) {
    if (!out) {
        g_create_error = "w4a16_dec_new: null out pointer";
        return 1;
    }
    *out = nullptr;
    int count = 0;
    cudaError_t e = cudaGetDeviceCount(&count);
    if (e != cudaSuccess || count == 0) {
        g_create_error = std::string("w4a16_dec_new: no CUDA device: ") + cudaGetErrorString(e);
        cudaGetLastError();
        return 1;
    }
    if (device < 0 || device >= count) {
        g_create_error = "w4a16_dec_new: device ordinal out of range";
        return 1;
    }
    e = cudaSetDevice(device);
    if (e != cudaSuccess) {
        g_create_error = std::string("w4a16_dec_new: cudaSetDevice: ") + cudaGetErrorString(e);
        return 1;
    }
    cudaDeviceProp prop;
    e = cudaGetDeviceProperties(&prop, device);
    if (e != cudaSuccess) {
        g_create_error = std::string("w4a16_dec_new: device properties: ") + cudaGetErrorString(e);
        return 1;
    }
    if (prop.major != 10) {
        g_create_error = "w4a16_dec_new: this library is built for sm_100a (B200) only";
        return 1;
    }
    w4a16_dec* dec = new w4a16_dec();
    Dec& d = dec->d;
    d.device = device;
    d.sm_count = prop.multiProcessorCount;
    e = cudaStreamCreateWithFlags(&d.stream, cudaStreamNonBlocking);
    if (e == cudaSuccess) {
        e = cudaMalloc(&d.err_flag, 4 * sizeof(int));
    }
    if (e == cudaSuccess) {
        e = cudaMalloc(&d.gemm_status, sizeof(int));
    }
    if (e == cudaSuccess) {
        e = cudaMemset(d.gemm_status, 0, sizeof(int));
    }
    if (e == cudaSuccess) {
        e = w4::gemv_init_device();
        if (e == cudaSuccess) {
            e = w4::gemv_sk_init_device();
        }
        if (e == cudaSuccess) {
            e = w4::gemv_rb_init_device();
        }
    }
    if (e == cudaSuccess) {
        e = w4::gemm_init_device();
    }
    if (e == cudaSuccess) {
        e = w4::head_init_device();
    }
    if (e != cudaSuccess) {
        g_create_error = std::string("w4a16_dec_new: ") + cudaGetErrorString(e);
        delete dec;
        return 1;
    }
    if (d.ensure_scratch(1 << 20, 4096, d.stream)) {
        g_create_error = d.err;
        delete dec;
        return 1;
    }
    *out = dec;
    return 0;
}

void w4a16_dec_free(w4a16_dec* dec) {
    if (!dec) {
        return;
    }
    Dec& d = dec->d;
    cudaSetDevice(d.device);
    cudaDeviceSynchronize();
    d.free_moe();
    for (auto& kv : d.lins) {
        d.free_lin(kv.second);
    }
    d.lins.clear();
    if (d.head_q) {
        cudaFree(d.head_q);
        cudaFree(d.head_scale);
    }
    for (void* p : d.retired) {
        cudaFree(p);
    }
    d.retired.clear();
    if (d.part) {
        cudaFree(d.part);
    }
    if (d.counters) {
        cudaFree(d.counters);
    }
    if (d.err_flag) {
        cudaFree(d.err_flag);
    }
    if (d.gemm_status) {
        cudaFree(d.gemm_status);
    }
    if (d.dbg_buf) {
        cudaFree(d.dbg_buf);
    }
    for (int p = 0; p < w4::TP_MAX_WORLD; ++p) {
        if (d.tp_peer[p] && d.tp_peer[p] != d.tp_block) {
            cudaIpcCloseMemHandle(d.tp_peer[p]);
        }
    }
    if (d.tp_block) {
        cudaFree(d.tp_block);
    }
    if (d.xh) {
        cudaFree(d.xh);
    }
    if (d.x16) {
        cudaFree(d.x16);
    }
    if (d.pin) {
        cudaFreeHost(d.pin);
    }
    if (d.stage_dev) {
        cudaFree(d.stage_dev);
    }
    if (d.yh) {
        cudaFree(d.yh);
    }
    if (d.stream) {
        cudaStreamDestroy(d.stream);
    }
    delete dec;
}

const char* w4a16_last_error(const w4a16_dec* dec) {
    return dec ? dec->d.err.c_str() : g_create_error.c_str();
}

void* w4a16_stream(w4a16_dec* dec) { return dec ? (void*)dec->d.stream : nullptr; }

int w4a16_sync(w4a16_dec* dec) {
    cudaError_t e = cudaStreamSynchronize(dec->d.stream);
    if (e != cudaSuccess) {
        return dec->d.cuda_fail("sync", e);
    }
    return w4a16_kernel_status(dec);
}

int w4a16_debug_timeline(w4a16_dec* dec, long long* out, int max_slots) {
    Dec& d = dec->d;
    if (!d.dbg_buf) {
        return d.fail("w4a16: timeline is off; set_tuning(\"debug_timeline\", 1) first");
    }
    const int n = max_slots < w4::DBG_SLOTS ? max_slots : w4::DBG_SLOTS;
    cudaError_t e = cudaDeviceSynchronize();
    if (e == cudaSuccess) {
        e = cudaMemcpy(out, d.dbg_buf, (size_t)n * sizeof(long long), cudaMemcpyDeviceToHost);
    }
    return e == cudaSuccess ? 0 : d.cuda_fail("read timeline", e);
}

int w4a16_kernel_status(w4a16_dec* dec) {
    Dec& d = dec->d;
    int st = 0;
    cudaError_t e = cudaMemcpy(&st, d.gemm_status, sizeof(int), cudaMemcpyDeviceToHost);
    if (e != cudaSuccess) {
        return d.cuda_fail("read kernel status", e);
    }
    if (st != 0) {
        cudaMemset(d.gemm_status, 0, sizeof(int));
        // an abandoned launch may have left tickets taken and peers' sums unread
        if (d.counters) {
            cudaMemset(d.counters, 0, d.counters_cap * sizeof(unsigned));
        }
        // the exchange block of the fused all-reduce is NOT re-armed here: the peers may still be pushing into
        // it, and all ranks must restart from the same launch number (w4a16_tp_rearm, between two host barriers)
        return d.fail("w4a16: a bounded pipeline wait expired (role %d, step %d); results are invalid%s", st >> 16,
                      st & 0xFFFF,
                      d.tp_block ? "; call w4a16_tp_rearm on every rank before the next fused all-reduce" : "");
    }
    return 0;
}

unsigned long long w4a16_launch_count(w4a16_dec* dec) { return dec->d.launches; }

const char* w4a16_last_kernel(w4a16_dec* dec) { return dec->d.last_kernel.c_str(); }

int w4a16_set_tuning(w4a16_dec* dec, const char* key, int value) {
    Dec& d = dec->d;
    if (!strcmp(key, "gemv_rowblock_units")) {
        d.tune_gemv_rowblock_units = value ? 1 : 0;
        return 0;
    }
    if (!strcmp(key, "gemv_stages")) {
        if (value < 2 || value > 8) {
            return d.fail("w4a16 tuning: gemv_stages must be 2..8");
        }
        d.tune_gemv_stages = value;
        return 0;
    }
    if (!strcmp(key, "gemm_mt")) {
        if (value < 0 || value > 2) {
            return d.fail("w4a16 tuning: gemm_mt must be 0, 1 or 2");
        }
        d.tune_gemm_mt = value;
        return 0;
    }
    if (!strcmp(key, "gemm_ksplit")) {
        if (value < -1 || value > 16) {
            return d.fail("w4a16 tuning: gemm_ksplit must be -1..16");
        }
        d.tune_gemm_ksplit = value;
        return 0;
    }
    if (!strcmp(key, "gemm_tma_store")) {
        d.tune_gemm_tma_store = value != 0;
        return 0;
    }
    if (!strcmp(key, "gemv_cluster")) {
        d.tune_gemv_cluster = value != 0;
        return 0;
    }
    if (!strcmp(key, "gemv_rowblock")) {
        if (value < 0 || value > 2) {
            return d.fail("w4a16 tuning: gemv_rowblock must be 0, 1 or 2");
        }
        d.tune_gemv_rowblock = value;
        return 0;
    }
    if (!strcmp(key, "gemv_persistent")) {
        d.tune_gemv_persistent = value;   // 0 = never, 1 = up to 4 tokens (default), 2 = always
        return 0;
    }
    if (!strcmp(key, "gemv_sk_prefetch")) {
        if (value < 0 || value > 6) {
            return d.fail("w4a16 tuning: gemv_sk_prefetch must be 0..6");
        }
        d.tune_gemv_sk_prefetch = value;
        return 0;
    }
    if (!strcmp(key, "gemv_sk_stages")) {
        if (value < 2 || value > 6) {
            return d.fail("w4a16 tuning: gemv_sk_stages must be 2..6");
        }
        d.tune_gemv_sk_stages = value;
        return 0;
    }
    if (!strcmp(key, "gemv_warps")) {
        if (value != 8 && value != 16) {
            return d.fail("w4a16 tuning: gemv_warps must be 8 or 16");
        }
        d.tune_gemv_warps = value;
        return 0;
    }
    if (!strcmp(key, "debug_timeline")) {
        if (value && !d.dbg_buf) {
            cudaError_t e = cudaMalloc(&d.dbg_buf, w4::DBG_SLOTS * sizeof(long long));
            if (e != cudaSuccess) {
                return d.cuda_fail("alloc timeline buffer", e);
            }
            cudaMemset(d.dbg_buf, 0, w4::DBG_SLOTS * sizeof(long long));
        } else if (!value && d.dbg_buf) {
            cudaDeviceSynchronize();
            cudaFree(d.dbg_buf);
            d.dbg_buf = nullptr;
        }
        return 0;
    }
    if (!strcmp(key, "pdl")) {
        if (value < 0 || value > 2) {
            return d.fail("w4a16 tuning: pdl must be 0, 1 or 2");
        }
        d.tune_pdl = value;
        return 0;
    }
    if (!strcmp(key, "tp_wait_log2")) {
        if (value < 16 || value > 40) {
            return d.fail("w4a16 tuning: tp_wait_log2 must be 16..40");
        }
        d.tune_tp_wait_log2 = value;
        d.tp.wait_cycles = 1ll << value;
        return 0;
    }
    if (!strcmp(key, "gemv_subnormal")) {
        d.tune_gemv_subnormal = value != 0;
        return 0;
    }
    if (!strcmp(key, "gemv_ksplit")) {
        if (value < 0 || value > 1024) {
            return d.fail("w4a16 tuning: gemv_ksplit must be 0..1024");
        }
        d.tune_gemv_ksplit = value;
        return 0;
    }
    return d.fail("w4a16 tuning: unknown key %s", key);
}

int w4a16_check_shapes(size_t t, size_t qlen, size_t slen, size_t xlen, size_t n, size_t k, size_t group) {
    // crates/backend-gpu/src/rawcuda/gptq4.rs:31-48. The reference's extra t==1 limit
    // (k <= group*256, its GEMV keeps scales in shared memory, :51-56) does not apply here.
    if ((group != 128 && group != 64 && group != 32) || k % group != 0 || t == 0 || qlen != n * (k / 8) ||
        slen != n * (k / group) || xlen != t * k) {
        return 1;
    }
    return 0;
}

static int validate_upload(Dec& d, const char* name, size_t q_bytes, size_t s_bytes, int n, int k, int group) {
    if (!name || !*name) {
        return d.fail("w4a16 upload: empty name");
    }
    if (n <= 0 || k <= 0 || (group != 128 && group != 64 && group != 32) || k % group != 0) {
        return d.fail("w4a16 upload %s: unsupported n=%d k=%d group=%d", name, n, k, group);
    }
    if (q_bytes != (size_t)n * (size_t)(k / 2) || s_bytes != (size_t)n * (size_t)(k / group) * 2) {
        return d.fail("w4a16 upload %s: q=%zu s=%zu bytes do not match n=%d k=%d g%d", name, q_bytes, s_bytes, n, k,
                      group);
    }
    if (!w4::shape_ok(n, k, group)) {
        return d.fail("w4a16 upload %s: tiled layout needs n%%16==0 and k%%64==0 (n=%d k=%d)", name, n, k);
    }
    return 0;
}

namespace {
struct SliceFill {
    const unsigned char* q;
    const unsigned char* s;
};
void slice_fill(void* user, int which, size_t off, void* dst, size_t len) {
    const SliceFill* f = (const SliceFill*)user;
    memcpy(dst, (which == 0 ? f->q : f->s) + off, len);
}
}  // namespace

int w4a16_upload_lin_g(w4a16_dec* dec, const char* name, const void* q, size_t q_bytes, const void* s,
                       size_t s_bytes, int n, int k, int group, int scale_bf16) {
    Dec& d = dec->d;
    cudaSetDevice(d.device);
    if (int rc = validate_upload(d, name, q_bytes, s_bytes, n, k, group)) {
        return rc;
    }
    // streamed in 8 MiB row chunks: no second full copy of the linear on the device
    SliceFill f{(const unsigned char*)q, (const unsigned char*)s};
    return d.upload_stream(name, n, k, group, scale_bf16, slice_fill, &f);
}

int w4a16_upload_lin_g_dev(w4a16_dec* dec, const char* name, const void* q_dev, const void* s_dev, int n,
                           int k, int group, int scale_bf16) {
    Dec& d = dec->d;
    cudaSetDevice(d.device);
    if (n <= 0 || k <= 0) {
        return d.fail("w4a16 upload: bad shape");
    }
    if (int rc = validate_upload(d, name, (size_t)n * (size_t)(k / 2),
                                 (group == 128 || group == 64 || group == 32) && k % group == 0
                                     ? (size_t)n * (size_t)(k / group) * 2
                                     : 0,
                                 n, k, group)) {
        return rc;
    }
    // order after whatever produced q/s on the legacy default stream
    cudaDeviceSynchronize();
    return d.upload_common(name, q_dev, s_dev, n, k, group, scale_bf16);
}

static Lin* find_lin(Dec& d, const char* name) {
    auto it = d.lins.find(name ? name : "");
    if (it == d.lins.end()) {
        d.fail("w4a16: unknown linear %s", name ? name : "(null)");
        return nullptr;
    }
    return &it->second;
}

int w4a16_lin_spec(w4a16_dec* dec, const char* name, int* n, int* k, int* group) {
    Lin* l = find_lin(dec->d, name);
    if (!l) {
        return 1;
    }
    if (n) *n = l->n;
    if (k) *k = l->k;
    if (group) *group = l->group_src;
    return 0;
}

int w4a16_drop_lin(w4a16_dec* dec, const char* name) {
    Dec& d = dec->d;
    auto it = d.lins.find(name ? name : "");
    if (it == d.lins.end()) {
        return d.fail("w4a16: unknown linear %s", name ? name : "(null)");
    }
    cudaSetDevice(d.device);
    cudaDeviceSynchronize();
    d.free_lin(it->second);
    d.lins.erase(it);
    return 0;
}

size_t w4a16_weights_bytes(w4a16_dec* dec) { return dec->d.weights_bytes; }

int w4a16_unpack_lin(w4a16_dec* dec, const char* name, void* q_dev, void* s_dev, void* stream) {
    Dec& d = dec->d;
    Lin* l = find_lin(d, name);
    if (!l) {
        return 1;
    }
    if (l->out_mul != 1.0f) {
        return d.fail("w4a16 unpack %s: its bf16 scales are not f16 values (use w4a16_dequant_lin)", name);
    }
    cudaStream_t st = pick_stream(dec, stream);
    w4::launch_unpack_q(l->qt, (uint32_t*)q_dev, l->n, l->k, st);
    w4::launch_unpack_s(l->st, (uint16_t*)s_dev, l->n, l->k, l->group, l->group_src == 64 ? 2 : 1, st);
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? 0 : d.cuda_fail("unpack", e);
}

int w4a16_dequant_lin(w4a16_dec* dec, const char* name, void* out_dev, int out_kind, void* stream) {
    Dec& d = dec->d;
    Lin* l = find_lin(d, name);
    if (!l) {
        return 1;
    }
    w4::launch_dequant(l->qt, l->st, out_dev, l->n, l->k, l->group, out_kind == W4A16_OUT_F16, l->out_mul,
                       pick_stream(dec, stream));
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? 0 : d.cuda_fail("dequant", e);
}

int w4a16_sk_single_dev(w4a16_dec* dec, const char* name, const void* x16_dev, void* out_dev, int t,
                        int out_kind, void* stream) {
    Dec& d = dec->d;
    Lin* l = find_lin(d, name);
    if (!l) {
        return 1;
    }
    const Lin* ls[1] = {l};
    void* outs[1] = {out_dev};
    return d.gemv(ls, 1, x16_dev, outs, t, out_kind, pick_stream(dec, stream));
}

// ---- row-parallel tensor parallelism ----------------------------------------------------------------
// exchange block layout: [seq u32][done u32][pad -> 4096 B][2 parities x world sources x 8 x max_rows f32, all ones]
int w4a16_tp_create(w4a16_dec* dec, int rank, int world, int max_rows, void* handle_out64) {
    Dec& d = dec->d;
    if (world < 2 || world > w4::TP_MAX_WORLD || rank < 0 || rank >= world || max_rows < 16 ||
        max_rows > w4::TP_MAX_CTAS * 256) {
        return d.fail("w4a16 tp_create: rank=%d world=%d max_rows=%d unsupported (world 2..%d, rows <= %d)", rank, world,
                      max_rows, w4::TP_MAX_WORLD, w4::TP_MAX_CTAS * 256);
    }
    cudaSetDevice(d.device);
    cudaDeviceSynchronize();
    if (d.tp_block) {
        return d.fail("w4a16 tp_create: already created");
    }
    const size_t area = (size_t)max_rows * w4::GEMV_MAX_M;
    if (max_rows % 4 != 0) {
        return d.fail("w4a16 tp_create: max_rows must be a multiple of 4");
    }
    const size_t bytes = TP_HEADER + 2 * (size_t)world * area * sizeof(float);
    cudaError_t e = cudaMalloc(&d.tp_block, bytes);
    if (e == cudaSuccess) e = cudaMemset(d.tp_block, 0, TP_HEADER);
    if (e == cudaSuccess) e = cudaMemset((char*)d.tp_block + TP_HEADER, 0xff, bytes - TP_HEADER);   // the sentinel
    cudaIpcMemHandle_t h;
    if (e == cudaSuccess) e = cudaIpcGetMemHandle(&h, d.tp_block);
    if (e != cudaSuccess) {
        return d.cuda_fail("tp_create", e);
    }
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
    memcpy(handle_out64, &h, 64);
    d.tp = w4::TpComm{};
    d.tp.rank = rank;
    d.tp.world = world;
    d.tp.area_floats = (int)area;
    d.tp.max_rows = max_rows;
    d.tp.wait_cycles = 1ll << d.tune_tp_wait_log2;
    d.tp_max_rows = max_rows;
    d.tp_peer[rank] = d.tp_block;
    return 0;
}

int w4a16_tp_connect(w4a16_dec* dec, const void* handles_world_x64) {
    Dec& d = dec->d;
    if (!d.tp_block) {
        return d.fail("w4a16 tp_connect: call w4a16_tp_create first");
    }
    cudaSetDevice(d.device);
    for (int p = 0; p < d.tp.world; ++p) {
        if (p != d.tp.rank && d.tp_peer[p] == nullptr) {
            cudaIpcMemHandle_t h;
            memcpy(&h, (const char*)handles_world_x64 + 64 * p, 64);
            cudaError_t e = cudaIpcOpenMemHandle(&d.tp_peer[p], h, cudaIpcMemLazyEnablePeerAccess);
            if (e != cudaSuccess) {
                return d.cuda_fail("tp_connect: cudaIpcOpenMemHandle", e);
            }
        }
    }
    for (int p = 0; p < d.tp.world; ++p) {
        d.tp.buf[p] = (float*)((char*)d.tp_peer[p] + TP_HEADER);
    }
    unsigned* local = (unsigned*)d.tp_block;
    d.tp.seq = local;
    d.tp.done = local + 1;
    return 0;
}

int w4a16_tp_rearm(w4a16_dec* dec) {
    Dec& d = dec->d;
    if (!d.tp_block) {
        return d.fail("w4a16 tp_rearm: call w4a16_tp_create first");
    }
    cudaSetDevice(d.device);
    cudaError_t e = cudaDeviceSynchronize();
    const size_t data = 2 * (size_t)d.tp.world * d.tp.area_floats * sizeof(float);
    if (e == cudaSuccess) e = cudaMemset(d.tp_block, 0, TP_HEADER);                      // launch number and done count
    if (e == cudaSuccess) e = cudaMemset((char*)d.tp_block + TP_HEADER, 0xff, data);     // every word: not arrived
    if (e == cudaSuccess && d.counters) e = cudaMemset(d.counters, 0, d.counters_cap * sizeof(unsigned));
    if (e == cudaSuccess) e = cudaMemset(d.gemm_status, 0, sizeof(int));
    if (e == cudaSuccess) e = cudaDeviceSynchronize();
    return e == cudaSuccess ? 0 : d.cuda_fail("tp_rearm", e);
}

int w4a16_sk_single_allreduce(w4a16_dec* dec, const char* name, const void* x16_dev, void* out_dev, int t,
                              int out_kind, void* stream) {
    Dec& d = dec->d;
    Lin* l = find_lin(d, name);
    if (!l) {
        return 1;
    }
    const Lin* ls[1] = {l};
    void* outs[1] = {out_dev};
    return d.gemv(ls, 1, x16_dev, outs, t, out_kind, pick_stream(dec, stream), true);
}

int w4a16_sk_multi_dev(w4a16_dec* dec, const char* const* names, int n_seg, const void* x16_dev,
                       void* const* outs_dev, int t, int out_kind, void* stream) {
    Dec& d = dec->d;
    if (n_seg < 1 || n_seg > w4::GEMV_MAX_SEG) {
        return d.fail("w4a16 sk_multi: %d segments outside 1..%d", n_seg, w4::GEMV_MAX_SEG);
    }
    const Lin* ls[w4::GEMV_MAX_SEG];
    for (int i = 0; i < n_seg; ++i) {
        ls[i] = find_lin(d, names[i]);
        if (!ls[i]) {
            return 1;
        }
    }
    if (t > w4::GEMV_MAX_M) {
        // the small-batch band above the decode GEMV (batch decode and speculative verify run q|k|v and gate|up at up
        // to 32 rows: crates/backend-gpu/src/rawcuda/w4a16_dec/chains.rs:315-507): one GEMM per segment
        for (int i = 0; i < n_seg; ++i) {
            if (int rc = d.gemm(ls[i], x16_dev, outs_dev[i], t, out_kind, pick_stream(dec, stream))) {
                return rc;
            }
        }
        return 0;
    }
    return d.gemv(ls, n_seg, x16_dev, outs_dev, t, out_kind, pick_stream(dec, stream));
}

int w4a16_lin_forward(w4a16_dec* dec, const char* name, const void* x16_dev, void* dst_dev, int t,
                      int out_kind, void* stream) {
    Dec& d = dec->d;
    Lin* l = find_lin(d, name);
    if (!l) {
        return 1;
    }
    if (t < 1) {
        return d.fail("w4a16 lin_forward %s: t=%d", name, t);
    }
    cudaStream_t st = pick_stream(dec, stream);
    if (t <= w4::GEMV_MAX_M) {
        const Lin* ls[1] = {l};
        void* outs[1] = {dst_dev};
        return d.gemv(ls, 1, x16_dev, outs, t, out_kind, st);
    }
    return d.gemm(l, x16_dev, dst_dev, t, out_kind, st);
}

int w4a16_lin_forward_lane(w4a16_dec* dec, const char* name, const void* x16_dev, float* dst_dev, int t, void* stream) {
    Dec& d = dec->d;
    Lin* l = find_lin(d, name);
    if (!l) {
        return 1;
    }
    if (t < 1 || t > 65535) {
        return d.fail("w4a16 lin_forward_lane %s: t=%d", name, t);
    }
    w4::launch_lane_mirror(l->qt, l->st, x16_dev, dst_dev, l->n, l->k, l->group, t, l->out_mul, pick_stream(dec, stream));
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) {
        return d.cuda_fail("launch lane mirror", e);
    }
    d.last_kernel = "lane_mirror_kernel";
    d.launches++;
    return 0;
}

int w4a16_lin_forward_x32(w4a16_dec* dec, const char* name, const float* x32_dev, void* dst_dev, int t, int out_kind,
                          void* stream) {
    Dec& d = dec->d;
    Lin* l = find_lin(d, name);
    if (!l) {
        return 1;
    }
    if (t < 1) {
        return d.fail("w4a16 lin_forward_x32 %s: t=%d", name, t);
    }
    cudaStream_t st = pick_stream(dec, stream);
    const size_t xb = (size_t)t * l->k * 2;
    if (xb > d.x16_cap) {
        if (Dec::capturing(st)) {
            return d.fail("w4a16 lin_forward_x32: staging too small during graph capture; run the call once before capturing");
        }
        cudaDeviceSynchronize();
        if (d.x16) {
            d.retired.push_back(d.x16);   // a captured graph may still name it
        }
        d.x16 = nullptr;
        d.x16_cap = 0;
        cudaError_t e = cudaMalloc(&d.x16, xb);
        if (e != cudaSuccess) {
            return d.cuda_fail("alloc f16 staging", e);
        }
        d.x16_cap = xb;
    }
    w4::launch_cast_f16(x32_dev, d.x16, (size_t)t * l->k, st);
    d.launches++;
    return w4a16_lin_forward(dec, name, d.x16, dst_dev, t, out_kind, stream);
}

int w4a16_lin_forward_host(w4a16_dec* dec, const char* name, const void* x16_host, void* dst_host, int t,
                           int out_kind) {
    Dec& d = dec->d;
    Lin* l = find_lin(d, name);
    if (!l) {
        return 1;
    }
    if (t < 1) {
        return d.fail("w4a16 lin_forward_host %s: t=%d", name, t);
    }
    const size_t xb = (size_t)t * l->k * 2;
    const size_t yb = (size_t)t * l->n * (out_kind == W4A16_OUT_F16 ? 2 : 4);
    if (xb > d.xh_cap) {
        cudaDeviceSynchronize();
        if (d.xh) cudaFree(d.xh);
        d.xh = nullptr;
        d.xh_cap = 0;
        cudaError_t e = cudaMalloc(&d.xh, xb);
        if (e != cudaSuccess) return d.cuda_fail("alloc x staging", e);
        d.xh_cap = xb;
    }
    if (yb > d.yh_cap) {
        cudaDeviceSynchronize();
        if (d.yh) cudaFree(d.yh);
        d.yh = nullptr;
        d.yh_cap = 0;
        cudaError_t e = cudaMalloc(&d.yh, yb);
        if (e != cudaSuccess) return d.cuda_fail("alloc y staging", e);
        d.yh_cap = yb;
    }
    cudaError_t e = cudaMemcpyAsync(d.xh, x16_host, xb, cudaMemcpyHostToDevice, d.stream);
    if (e != cudaSuccess) return d.cuda_fail("copy x to device", e);
    if (int rc = w4a16_lin_forward(dec, name, d.xh, d.yh, t, out_kind, d.stream)) {
        return rc;
    }
    e = cudaMemcpyAsync(dst_host, d.yh, yb, cudaMemcpyDeviceToHost, d.stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(d.stream);
    return e == cudaSuccess ? 0 : d.cuda_fail("copy y to host", e);
}

int w4a16_gptq4_gemm(w4a16_dec* dec, const void* x16_host, int t, const void* q_host, const void* s_host,
                     int n, int k, int group, int scale_bf16, float* out_host) {
    Dec& d = dec->d;
    if (n <= 0 || k <= 0 || t <= 0 || (group != 128 && group != 64 && group != 32) || k % group != 0) {
        return d.fail("gptq4: shape contract violated n=%d k=%d t=%d group=%d", n, k, t, group);
    }
    static const char* TMP = "\x01gptq4.tmp";
    if (int rc = w4a16_upload_lin_g(dec, TMP, q_host, (size_t)n * (k / 2), s_host, (size_t)n * (k / group) * 2, n,
                                    k, group, scale_bf16)) {
        return rc;
    }
    int rc = w4a16_lin_forward_host(dec, TMP, x16_host, out_host, t, W4A16_OUT_F32);
    std::string keep = d.err;
    w4a16_drop_lin(dec, TMP);
    if (rc) d.err = keep;
    return rc;
}

int w4a16_capture_begin(w4a16_dec* dec) {
    cudaError_t e = cudaStreamBeginCapture(dec->d.stream, cudaStreamCaptureModeThreadLocal);
    return e == cudaSuccess ? 0 : dec->d.cuda_fail("cudaStreamBeginCapture", e);
}

int w4a16_capture_end(w4a16_dec* dec, void** graph_exec_out) {
    Dec& d = dec->d;
    cudaGraph_t g = nullptr;
    cudaError_t e = cudaStreamEndCapture(d.stream, &g);
    if (e != cudaSuccess) {
        return d.cuda_fail("cudaStreamEndCapture", e);
    }
    cudaGraphExec_t ex = nullptr;
    e = cudaGraphInstantiate(&ex, g, 0);
    cudaGraphDestroy(g);
    if (e != cudaSuccess) {
        return d.cuda_fail("cudaGraphInstantiate", e);
    }
    e = cudaGraphUpload(ex, d.stream);
    if (e != cudaSuccess) {
        cudaGraphExecDestroy(ex);
        return d.cuda_fail("cudaGraphUpload", e);
    }
    *graph_exec_out = (void*)ex;
    return 0;
}

int w4a16_graph_launch(w4a16_dec* dec, void* graph_exec) {
    cudaError_t e = cudaGraphLaunch((cudaGraphExec_t)graph_exec, dec->d.stream);
    return e == cudaSuccess ? 0 : dec->d.cuda_fail("cudaGraphLaunch", e);
}

int w4a16_graph_destroy(w4a16_dec* dec, void* graph_exec) {
    cudaError_t e = cudaGraphExecDestroy((cudaGraphExec_t)graph_exec);
    return e == cudaSuccess ? 0 : dec->d.cuda_fail("cudaGraphExecDestroy", e);
}

int w4a16_graph_step_host(w4a16_dec* dec, void* graph_exec, const void* x_host, void* x_dev,
                          size_t x_bytes, const void* y_dev, void* y_host, size_t y_bytes) {
    Dec& d = dec->d;
    cudaError_t e = cudaMemcpyAsync(x_dev, x_host, x_bytes, cudaMemcpyHostToDevice, d.stream);
    if (e == cudaSuccess) e = cudaGraphLaunch((cudaGraphExec_t)graph_exec, d.stream);
    if (e == cudaSuccess) e = cudaMemcpyAsync(y_host, y_dev, y_bytes, cudaMemcpyDeviceToHost, d.stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(d.stream);
    return e == cudaSuccess ? 0 : d.cuda_fail("graph step", e);
}

}  // extern "C"
