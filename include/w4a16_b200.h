/*
 * libw4a16_b200 -- C ABI of the B200-native W4A16 matmul path.
 *
 * Drop-in boundary for the linear / MoE call sites of LLM170's crates/backend-gpu: every entry
 * point below names the reference interface it replaces (file:line inside the reference tree).
 * Conventions shared by all calls:
 *   - plain pointers and sizes only; `stream` is a cudaStream_t passed as void* (NULL = the
 *     decoder's own stream, like `cc.stream` in the reference);
 *   - return 0 on success, non-zero on error; the message is read with w4a16_last_error().  The
 *     reference returns Result<_, String> from every call and never panics across the boundary
 *     (crates/backend-gpu/src/rawcuda/ffi.rs:18-40);
 *   - a decoder is bound to one device and is not thread-safe (the reference's W4a16Dec is Send
 *     but not Sync: crates/backend-gpu/src/rawcuda/w4a16_dec/mod.rs:626);
 *   - weights and scratch are owned by the decoder; activations and outputs by the caller;
 *   - forward calls launch asynchronously, allocate nothing once warmed, and may be captured in a
 *     CUDA graph (crates/backend-gpu/src/rawcuda/ctx/graph.rs:4-65).
 * Weight format at the boundary (compressed-tensors pack-quantized, crates/core/src/w4a16.rs:124-175):
 *   q: little-endian u32 [n][k/8], element i of a row = nibble at bits 4*(i&7) of word i>>3, value q+8
 *   s: f16 (or bf16) [n][k/group], group in {128, 64, 32};  dequantised weight = (nibble-8)*scale.
 */
#ifndef W4A16_B200_H
#define W4A16_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define W4A16_API __attribute__((visibility("default")))
#else
#define W4A16_API
#endif

typedef struct w4a16_dec w4a16_dec;
/* a mapped safetensors archive (w4a16_st_open) */
typedef struct w4a16_st w4a16_st;
/* chunk callback of w4a16_upload_lin_g_stream */
typedef void (*w4a16_fill_fn)(void* user, int which, size_t off, void* dst, size_t len);

/* Output element type of a forward call. The reference writes f32 (dst of lin_forward). */
#define W4A16_OUT_F32 0
#define W4A16_OUT_F16 1

/* ---- lifetime ---------------------------------------------------------------------------- */

/* W4a16Dec::new_dev (crates/backend-gpu/src/rawcuda/w4a16_dec/mod.rs:654) + CudaCtx::new_dev
 * (crates/backend-gpu/src/rawcuda/ctx/mod.rs:101-178): binds the
 * device's primary context, creates the decoder stream and the split-K scratch. */
W4A16_API int w4a16_dec_new(int device, w4a16_dec** out);
/* CudaCtx::free_all (crates/backend-gpu/src/rawcuda/ctx/mem.rs:19): frees weights, scratch, stream. */
W4A16_API void w4a16_dec_free(w4a16_dec* dec);
/* Text of the last error on `dec` (or of the last failed w4a16_dec_new when dec is NULL): the
 * String of the reference's Err (crates/backend-gpu/src/rawcuda/ffi.rs:18-40). */
W4A16_API const char* w4a16_last_error(const w4a16_dec* dec);
/* The decoder's stream (CudaCtx.stream, crates/backend-gpu/src/rawcuda/ctx/mod.rs:60-75), as a
 * cudaStream_t. */
W4A16_API void* w4a16_stream(w4a16_dec* dec);
/* CudaCtx::sync (crates/backend-gpu/src/rawcuda/ctx/mod.rs:407). */
W4A16_API int w4a16_sync(w4a16_dec* dec);
/* Synchronises the device and reports whether a kernel gave up on a bounded wait since the last
 * check (0 = none). Every device-side wait in this library has an iteration limit and records a
 * status word instead of hanging; the reference's only guard is its host watchdog
 * (crates/diag/src/watchdog.rs:46-90). w4a16_sync() includes this check. */
W4A16_API int w4a16_kernel_status(w4a16_dec* dec);
/* Diagnostic: after set_tuning("debug_timeline", 1), every CTA of a decode GEMV stamps the global
 * nanosecond timer at its pipeline events (entry, previous kernel complete, x staged, main loop start,
 * main loop end, exit; then its SM id, unit count, and the steps of the cross-CTA reduce) into a device buffer
 * laid out [launch number mod 64][CTA < 384][16]; this copies up to max_slots entries out.
 * Plays the role of the reference's per-launch event profiler
 * (crates/backend-gpu/src/rawcuda/ctx/prof.rs:56-131) at a finer grain. */
W4A16_API int w4a16_debug_timeline(w4a16_dec* dec, long long* out, int max_slots);
/* Kernels launched by forward calls since creation: the launch counter the reference keeps in
 * HOST_LAUNCH_CALLS (crates/backend-gpu/src/rawcuda/ctx/mod.rs:10-11,311-315). */
W4A16_API unsigned long long w4a16_launch_count(w4a16_dec* dec);
/* Name of the kernel instantiation the last forward call on `dec` launched (e.g. "gemv_sk_kernel<128,true>"),
 * for reports; the reference names its kernels by fatbin symbol
 * (crates/backend-gpu/src/rawcuda/gptq4.rs:60-70). Valid until the next forward call. */
W4A16_API const char* w4a16_last_kernel(w4a16_dec* dec);
/* Kernel-selection knobs, the analogue of the reference's LLM170_* environment flags
 * (crates/diag/src/flag.rs:3-27). Keys: "gemv_persistent" (which form of the decode GEMV runs: 1 = default,
 * two persistent CTAs per SM with equal ranges of work for up to 4 tokens and the (row block, K split) grid
 * above that; 2 = always persistent; 0 = never), "tp_wait_log2" (16..40, default 31: the fused all-reduce gives up
 * on its peers after 2^n cycles), "gemv_sk_stages" (2..6) and "gemv_sk_prefetch" (0..6): ring
 * stages of the persistent form and how many of them are requested before the previous kernel of the stream is
 * complete; "gemv_rowblock" (1 = default: up to four tokens of a 128-channel-group linear of at most 48 MB and K <= 6144 run on CTAs that own whole rows, without scratch or tickets -- a 16-warp kernel when all 32-row units are resident at once and x fits beside the weights in shared memory, else an 8-warp kernel up to tokens x K <= 11264 and the (row block, K split) form beyond; 2 = whatever the size; 0 = never), "gemv_rowblock_units" (1 = default; 0 = never the 16-warp kernel); the remaining gemv_* keys tune the (row block, K split) form: "gemv_ksplit" (0 = automatic),
 * "gemv_stages" (16 KB weight stages in flight per CTA, 2..8), "gemv_warps" (consumer warps per CTA, 8 or 16), "gemv_cluster" (1 = default: 2..8 K splits of a row
 * block run as a thread-block cluster and reduce through distributed shared memory),
 * "gemv_subnormal" (1 = default arithmetic, 0 = exact nibble-8 operands), "gemm_mt" (128-token blocks per prefill GEMM tile: 0 = automatic, 1, 2), "gemm_ksplit" (K splits of the GEMM tiles: 0 = automatic -- all tiles when they are few, the tiles of an incomplete last wave otherwise; -1 = never; 1..16 = every tile), "gemm_tma_store" (1 = default: whole dense tiles leave through shared memory and TMA stores; 0 = per-lane stores), "debug_timeline" (0/1, see w4a16_debug_timeline), "pdl" (1 = default: kernels are
 * launched with programmatic stream serialization and prefetch weights while the previous kernel of
 * the stream drains; 2 = the next kernel may start as soon as this one is resident; 0 = ordinary launches). */
W4A16_API int w4a16_set_tuning(w4a16_dec* dec, const char* key, int value);

/* ---- weights ----------------------------------------------------------------------------- */

/* gptq4::check_shapes (crates/backend-gpu/src/rawcuda/gptq4.rs:31-58): validates lengths (in
 * elements: q u32 words, s u16, x u16) against n, k, t, group. Needs no device. 0 = accepted. */
W4A16_API int w4a16_check_shapes(size_t t, size_t qlen, size_t slen, size_t xlen, size_t n, size_t k, size_t group);

/* W4a16Dec::upload_lin_g (crates/backend-gpu/src/rawcuda/w4a16_dec/upload.rs:15-65) followed by
 * the repack of upload_lin_marlin (:99-179): copies q (n*k/2 bytes) and s (n*(k/group)*2 bytes)
 * from HOST memory, re-tiles them on the device into the library's single resident layout and
 * registers the linear under `name`, replacing (and freeing) a previous one of that name. */
W4A16_API int w4a16_upload_lin_g(w4a16_dec* dec, const char* name, const void* q, size_t q_bytes, const void* s,
                       size_t s_bytes, int n, int k, int group, int scale_bf16);
/* Same, with q and s already in DEVICE memory in the boundary format (used when weights are
 * produced on the device; the reference has no such variant). */
W4A16_API int w4a16_upload_lin_g_dev(w4a16_dec* dec, const char* name, const void* q_dev, const void* s_dev, int n,
                           int k, int group, int scale_bf16);
/* W4a16Dec::upload_lin_g_stream (crates/backend-gpu/src/rawcuda/w4a16_dec/upload.rs:1643; experts
 * upload_experts_resident_streamed, :1021-1082): the caller does not hold the linear as one host slice but fills
 * chunks on request. `fill(user, which, off, dst, len)` must write bytes [off, off+len) of q (which == 0) or of s
 * (which == 1) to dst, a pinned buffer of the decoder; it is called for whole rows, in 8 MiB chunks, and twice over
 * the scales when they are bf16. Every chunk is re-tiled into place as it arrives, so the load needs neither the
 * whole host slice nor a second copy of the linear on the device (w4a16_upload_lin_g is built on this call). */
W4A16_API int w4a16_upload_lin_g_stream(w4a16_dec* dec, const char* name, int n, int k, int group, int scale_bf16,
                                        w4a16_fill_fn fill, void* user);
/* W4a16Dec::lin_spec (crates/backend-gpu/src/rawcuda/w4a16_dec/mod.rs:1193): n and k, plus the
 * group size; non-zero if `name` is unknown. */
W4A16_API int w4a16_lin_spec(w4a16_dec* dec, const char* name, int* n, int* k, int* group);
/* Frees one linear (what replacing a name does in
 * crates/backend-gpu/src/rawcuda/w4a16_dec/upload.rs:52-55). */
W4A16_API int w4a16_drop_lin(w4a16_dec* dec, const char* name);
/* Bytes of device memory held by weights (weights_bytes,
 * crates/backend-gpu/src/rawcuda/w4a16_dec/upload.rs:51). */
W4A16_API size_t w4a16_weights_bytes(w4a16_dec* dec);

/* Inverse of the re-tiling: writes the boundary-format q (u32 [n][k/8]) and s (f16 [n][k/group])
 * back into DEVICE buffers. Role of the `unrepack` helper in crates/core/src/marlin.rs:75-105. */
W4A16_API int w4a16_unpack_lin(w4a16_dec* dec, const char* name, void* q_dev, void* s_dev, void* stream);
/* Element-wise dequantisation of a resident linear into a DEVICE buffer [n][k]:
 * out_kind W4A16_OUT_F32 -> (nibble-8)*scale exactly as crates/core/src/matmul/cpu.rs:167-194;
 * W4A16_OUT_F16 -> that value rounded once to f16, the operand the tensor-core GEMM multiplies. */
W4A16_API int w4a16_dequant_lin(w4a16_dec* dec, const char* name, void* out_dev, int out_kind, void* stream);

/* ---- checkpoints and the tile cache -------------------------------------------------------- */

/* StArchive::open (crates/core/src/st.rs:115-290) + the triple scan of W4a16Model::open
 * (crates/core/src/w4a16.rs:108-191): maps a .safetensors file, or every model*.safetensors of a directory,
 * checks each header entry (dtype, shape x element size == data_offsets, inside the file) and collects the
 * linears: every `<base>.weight_packed` (I32 [n, k/8]) with `<base>.weight_scale` (F16 / BF16 [n, k/group],
 * group 32, 64 or 128) and `<base>.weight_shape` (I64 [2] = n, k). Needs no device. Errors: w4a16_st_error(). */
W4A16_API int w4a16_st_open(const char* path, w4a16_st** out);
W4A16_API void w4a16_st_close(w4a16_st* st);
W4A16_API const char* w4a16_st_error(void);
/* W4a16Model::lins (crates/core/src/w4a16.rs:170-175): number of linears, and the i-th one in name order. */
W4A16_API int w4a16_st_lin_count(const w4a16_st* st);
W4A16_API int w4a16_st_lin_at(const w4a16_st* st, int i, char* base_out, size_t cap, int* n, int* k, int* group,
                              int* scale_bf16);
/* 64-bit FNV-1a over a linear's shape, packed weights and scales: names what a cache file was made from. It has
 * no counterpart in the reference, which keeps no weight cache (its prebuilt kernel binaries are guarded by a
 * hash manifest in the same spirit, scripts/preflight.sh). */
W4A16_API int w4a16_st_lin_tag(const w4a16_st* st, const char* base, uint64_t* tag);
/* upload_model's per-linear step (crates/server/src/gpu_engine/upload.rs:264-305): streams linear `base` of the
 * archive to the device under `name`, straight from the mapped file. */
W4A16_API int w4a16_upload_lin_st(w4a16_dec* dec, const char* name, const w4a16_st* st, const char* base);
/* Tile cache (no counterpart in the reference, which re-runs its host repack at every load:
 * crates/backend-gpu/src/rawcuda/w4a16_dec/upload.rs:99-179). save writes the resident tiles of `name` with a
 * header (shape, groups, layout version, source_tag); load puts a linear back with plain host-to-device copies --
 * no staging copy, no repack -- and refuses a file of another layout version or another source_tag. */
W4A16_API int w4a16_save_lin_cache(w4a16_dec* dec, const char* name, const char* path, uint64_t source_tag);
W4A16_API int w4a16_load_lin_cache(w4a16_dec* dec, const char* name, const char* path, uint64_t source_tag);

/* ---- linear forward ---------------------------------------------------------------------- */

/* W4a16Dec::lin_forward (crates/backend-gpu/src/rawcuda/w4a16_dec/kernels/mod.rs:121-144):
 * dst[t][n] = x16[t][k] * W^T. x16 is f16 row-major on the device, dst f32 or f16. Chooses the
 * split-K GEMV for t <= 8 and the tensor-core GEMM above (the reference switches at t > 8 too:
 * crates/backend-gpu/src/rawcuda/w4a16_dec/prefill.rs:81-345). */
W4A16_API int w4a16_lin_forward(w4a16_dec* dec, const char* name, const void* x16_dev, void* dst_dev, int t,
                      int out_kind, void* stream);
/* lin_forward for callers that hold f32 activations, as the reference's FFMA paths do (x f32 holding f16 values,
 * crates/backend-gpu/src/rawcuda/w4a16_dec/kernels/gemv.rs:4-38; cast kernel w4a16_cast_f16,
 * crates/backend-gpu/src/rawcuda/assets/moepp.cu:36-51): rounds x32[t][k] to f16 into a staging buffer of the
 * decoder (grown outside graph capture only), then runs w4a16_lin_forward on it. */
W4A16_API int w4a16_lin_forward_x32(w4a16_dec* dec, const char* name, const float* x32_dev, void* dst_dev, int t,
                                    int out_kind, void* stream);
/* The parity-gate kernel: dst[t][n] f32 computed in the lane order of crates/core/src/quant/lane.rs:2-70 (64 f32
 * lane accumulators, un-fused multiply and add, f64 tree), bit-identical to the CPU lane dot for every t. Takes the
 * place of the reference's FFMA mirror w4a16_gemm_g128 / w4a16_gemm_g32_bf16
 * (crates/backend-gpu/src/rawcuda/assets/gptq4.cu:825-951), which the gate
 * crates/server/src/probes/w4a16/gates.rs:108-138 compares bit for bit. A checking tool, not a fast path. */
W4A16_API int w4a16_lin_forward_lane(w4a16_dec* dec, const char* name, const void* x16_dev, float* dst_dev, int t,
                                     void* stream);

/* ---- int8 lm-head ------------------------------------------------------------------------- */
/* W4a16Dec::upload_head (crates/backend-gpu/src/rawcuda/w4a16_dec/upload.rs:1472-1569): w is the bf16 [n][k] matrix
 * on the host; every row is quantised to int8 with scale = absmax/127 (1 for a zero row) and
 * q = round-half-away(v / scale) clamped to +-127 -- on the device, bit-identical to the host recipe.
 * k must be a multiple of 64.  Replaces an earlier lm-head of the decoder. */
W4A16_API int w4a16_upload_head(w4a16_dec* dec, const void* w_bf16_host, size_t bytes, int n, int k);
/* head_n / head_k of the decoder (crates/backend-gpu/src/rawcuda/w4a16_dec/upload.rs:1564-1568). */
W4A16_API int w4a16_head_spec(w4a16_dec* dec, int* n, int* k);
/* Reads the quantised rows (int8 [n][k], two's complement) and the f32 row scales back; scale_host may be NULL.
 * For tests of the quantiser; no counterpart in the reference. */
W4A16_API int w4a16_head_unpack(w4a16_dec* dec, void* q_host, void* scale_host);
/* head_gemv_launch / head_gemv_t_launch (crates/backend-gpu/src/rawcuda/w4a16_dec/kernels/gemv.rs:64-110; kernels
 * w4a16_gemv_i8, w4a16_gemv_i8_t, crates/backend-gpu/src/rawcuda/assets/head.cu:100-225):
 * out[t][n] f32 = (sum_k q[n][k] * x[t][k]) * scale[n] for x f32 [t][k] on the device, 1 <= t <= 16.
 * The sum runs on the tensor cores with x split into two f16 planes (|x| must lie inside the f16 range);
 * it agrees with the reference's f32 lane sum within 1e-5 of sum_k |q x| * scale (both are f32 sums in different orders). */
W4A16_API int w4a16_head_forward(w4a16_dec* dec, const float* x32_dev, float* out_dev, int t, void* stream);
/* W4a16Dec::sk_single_dev (crates/backend-gpu/src/rawcuda/w4a16_dec/kernels/decode.rs:89-127):
 * the decode GEMV on one linear, t in 1..8. */
W4A16_API int w4a16_sk_single_dev(w4a16_dec* dec, const char* name, const void* x16_dev, void* out_dev, int t,
                        int out_kind, void* stream);
/* W4a16Dec::sk_multi_dev (crates/backend-gpu/src/rawcuda/w4a16_dec/kernels/decode.rs:23-57): up to
 * four linears that share x and k (q|k|v, gate|up) in ONE launch for t <= 8; outs[i] is [t][n_i]. Above 8 rows
 * (gemv_multi_t_dev of the batch-decode chain, crates/backend-gpu/src/rawcuda/w4a16_dec/kernels/gemv.rs:272-300)
 * each segment runs through the tensor-core GEMM. */
W4A16_API int w4a16_sk_multi_dev(w4a16_dec* dec, const char* const* names, int n_seg, const void* x16_dev,
                       void* const* outs_dev, int t, int out_kind, void* stream);
/* The decode GEMV of w4a16_sk_single_dev for hosts that must not allocate device memory (an engine that
 * owns the whole memory budget and forbids library allocations after start-up, or a decode loop in
 * which a cudaMalloc -- a device-wide synchronisation -- may never occur). It has no counterpart in the
 * reference. The split-K scratch lives in an 8 MiB + 16 KiB array inside the library's device image
 * (held by every GPU that loads the library, until exit), so this call allocates nothing. A shape whose
 * launch needs more than 8 MiB of partial sums (8 KB per K split and 256-row block) or more than 4096
 * row blocks is rejected with an error. All calls share the array: calls that overlap on the GPU race;
 * calls on one stream are safe. The first call on a device resolves the array's address
 * (cudaGetSymbolAddress) and must be made outside stream capture, with that device current. */
W4A16_API int w4a16_sk_single_static(w4a16_dec* dec, const char* name, const void* x16_dev, void* out_dev, int t,
                                     int out_kind, void* stream);
/* Host-buffer form of lin_forward: copies x from HOST (pinned or pageable) memory, runs the
 * linear, copies dst back and synchronises. The end-to-end call a host engine makes per step
 * (the reference's host round trip: Gptq4::gemm, crates/backend-gpu/src/rawcuda/gptq4.rs:99-189,
 * with the weights already resident as in W4a16Dec). */
W4A16_API int w4a16_lin_forward_host(w4a16_dec* dec, const char* name, const void* x16_host, void* dst_host, int t,
                           int out_kind);
/* Gptq4::gemm (crates/backend-gpu/src/rawcuda/gptq4.rs:99-189): everything from HOST memory --
 * uploads q and s, runs x[t][k] through the linear, returns f32 [t][n], frees the weights. */
W4A16_API int w4a16_gptq4_gemm(w4a16_dec* dec, const void* x16_host, int t, const void* q_host, const void* s_host,
                     int n, int k, int group, int scale_bf16, float* out_host);

/* ---- row-parallel tensor parallelism (no counterpart in the reference, which has no collective:
 *      crates/server/src/main.rs:245-247) ------------------------------------------------------ */

/* Allocates this rank's exchange block (a launch counter and, for each of two launch parities and each source
 * rank, a receive area of 8 x max_rows f32 partial sums; max_rows a multiple of 4) and returns its 64-byte CUDA
 * IPC handle. rank/world describe the tensor-parallel group on one node
 * (world 2..8, one process per GPU). The reference has no such variant. */
W4A16_API int w4a16_tp_create(w4a16_dec* dec, int rank, int world, int max_rows, void* handle_out64);
/* Maps the peers' exchange blocks: `handles` holds world x 64 bytes, the handles of all ranks in rank
 * order (exchanged by the host, e.g. over its process group). The reference has no such variant. */
W4A16_API int w4a16_tp_connect(w4a16_dec* dec, const void* handles_world_x64);
/* Puts this rank's exchange block back into its initial state (launch number 0, every word "not arrived") and
 * clears the kernel status. To be called by EVERY rank after any rank saw a fused all-reduce give up
 * (w4a16_kernel_status / w4a16_sync returned an error), between two host barriers: barrier, rearm, barrier.
 * The ranks then agree on the launch number again and no stale word of the abandoned launch survives.
 * The reference has no such variant. */
W4A16_API int w4a16_tp_rearm(w4a16_dec* dec);
/* Row-parallel decode GEMV with the all-reduce fused into the kernel: each rank holds a K slice of the
 * linear (whole scale groups), x16 is that slice of the activations, and out receives the SUM over ranks
 * of the partial products -- the kernel that reduces the split-K partials also pushes the local sums into
 * every peer's receive area with peer stores over NVLink, waits (bounded) until the peers' sums have arrived
 * in its own and adds them in rank order. The wait is bounded (about a second, "tp_wait_log2"): ranks whose
 * hosts drift further apart than that give up, w4a16_kernel_status reports it, and all ranks must then call
 * w4a16_tp_rearm. Every rank must make the same sequence of these calls. Replaces sk_single_dev + an NCCL all-reduce for o_proj / down
 * (the reference runs them on one GPU: crates/backend-gpu/src/rawcuda/w4a16_dec/kernels/decode.rs:89-127). */
W4A16_API int w4a16_sk_single_allreduce(w4a16_dec* dec, const char* name, const void* x16_dev, void* out_dev, int t,
                                        int out_kind, void* stream);

/* ---- MoE ---------------------------------------------------------------------------------- */

/* W4a16Dec::set_moe (crates/backend-gpu/src/rawcuda/w4a16_dec/upload.rs:795-812): expert count, top-k,
 * expert intermediate size, hidden size and quantisation group of the expert linears. The last two
 * arguments name the experts resident on THIS decoder, [expert_first, expert_first+expert_count):
 * all of them on one GPU, 128/G per GPU under expert parallelism (the reference keeps all experts on
 * one device: crates/backend-gpu/src/rawcuda/w4a16_dec/moe/mod.rs:77-101). */
W4A16_API int w4a16_set_moe(w4a16_dec* dec, int n_experts, int top_k, int moe_ffn, int hidden, int group,
                            int expert_first, int expert_count);
/* upload_experts_resident_streamed + build_marlin_moe_arenas
 * (crates/backend-gpu/src/rawcuda/w4a16_dec/upload.rs:1021-1082,1116-1235): the local experts of one
 * layer from HOST memory, in the boundary format, stacked expert-major: w13 = gate rows then up rows
 * per expert, q u32 [count][2*ffn][hidden/8], s [count][2*ffn][hidden/group]; w2 = down,
 * q [count][hidden][ffn/8], s [count][hidden][ffn/group]. */
W4A16_API int w4a16_upload_experts(w4a16_dec* dec, int layer, const void* w13_q, const void* w13_s, const void* w2_q,
                                   const void* w2_s, int scale_bf16);
/* Same with the four arrays already in DEVICE memory (the reference has no such variant). */
W4A16_API int w4a16_upload_experts_dev(w4a16_dec* dec, int layer, const void* w13_q, const void* w13_s,
                                       const void* w2_q, const void* w2_s, int scale_bf16);
/* w4a16_moe_topk_t (crates/backend-gpu/src/rawcuda/assets/moe.cu:686-759; host mirror moe_topk,
 * crates/backend-gpu/src/rawcuda/w4a16_dec/mod.rs:168-185): softmax over f32 logits [t][n_experts],
 * top-k with lower-index tie-break, weights renormalised over the k picked. idx int32 [t][k], wt f32 [t][k]. */
W4A16_API int w4a16_moe_topk(w4a16_dec* dec, const float* logits_dev, int* idx_dev, float* wt_dev, int t, void* stream);
/* W4a16Dec::moe_ffn_dev_t (crates/backend-gpu/src/rawcuda/w4a16_dec/moe/mod.rs:263-447) on the resident
 * grouped-GEMM path (crates/backend-gpu/src/rawcuda/w4a16_dec/kernels/marlin_moe.rs:290-422):
 * y[t][hidden] = sum over the token's top-k experts of w * down_e( silu(gate_e x) * up_e x ), restricted to
 * the local experts (under expert parallelism the caller sums y over ranks). router logits f32 [t][n_experts]
 * come from the caller (a plain GEMM outside this path); x16 f16 [t][hidden]; y f32 or f16. */
W4A16_API int w4a16_moe_ffn(w4a16_dec* dec, int layer, const float* router_logits_dev, const void* x16_dev, void* y_dev,
                            int t, int out_kind, void* stream);

/* ---- graph capture ----------------------------------------------------------------------- */

/* CudaCtx::capture_begin / capture_end / graph_instantiate / graph_launch / graph destroy
 * (crates/backend-gpu/src/rawcuda/ctx/graph.rs:4-85) on the decoder's stream. A forward call
 * that would have to grow scratch during capture fails instead; run it once un-captured first
 * (the reference's warm_for_capture, crates/backend-gpu/src/rawcuda/ctx/mod.rs:379-384). */
W4A16_API int w4a16_capture_begin(w4a16_dec* dec);
W4A16_API int w4a16_capture_end(w4a16_dec* dec, void** graph_exec_out);
W4A16_API int w4a16_graph_launch(w4a16_dec* dec, void* graph_exec);
W4A16_API int w4a16_graph_destroy(w4a16_dec* dec, void* graph_exec);
/* One host-driven step over a captured chain, the shape of W4a16Dec::forward_device_argmax
 * (crates/backend-gpu/src/rawcuda/w4a16_dec/graphs.rs:202): copies x_bytes from HOST x_host to
 * DEVICE x_dev, replays the graph, copies y_bytes from DEVICE y_dev to HOST y_host, synchronises. */
W4A16_API int w4a16_graph_step_host(w4a16_dec* dec, void* graph_exec, const void* x_host, void* x_dev,
                                    size_t x_bytes, const void* y_dev, void* y_host, size_t y_bytes);

#ifdef __cplusplus
}
#endif
#endif /* W4A16_B200_H */
