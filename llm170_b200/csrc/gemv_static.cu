// Decode GEMV for callers that must not allocate device memory.
//
// w4a16_sk_single_dev() keeps its split-K scratch (partial sums and arrival tickets) in buffers the
// decoder grows with cudaMalloc when a larger shape first shows up.  Some hosts cannot tolerate that: an
// engine that hands its whole device-memory budget to its own pool and forbids allocations by libraries
// after start-up, or a latency-critical decode loop where a cudaMalloc (which synchronises the device)
// must never happen.  w4a16_sk_single_static() runs the same kernel with the scratch placed in a
// fixed-size array that is part of this library's device image, so the call allocates nothing at all.
//
// Limits and rules:
//   * the scratch a launch needs -- 8 KB per (K split, 256-row block) plus one ticket per row block -- must
//     fit STATIC_PART_BYTES / STATIC_TICKETS; otherwise the call fails with a message and launches nothing;
//   * the array exists once per GPU that loads the library, and stays until the process exits;
//   * every call shares it.  The array keeps whatever the previous call left; the partial sums are fully
//     rewritten before they are read and the tickets a launch uses are cleared on the stream before it,
//     so consecutive calls on one stream are safe, but two calls that overlap on the GPU (different
//     streams) race on it;
//   * the first call on a device looks up the array's device address (cudaGetSymbolAddress with that
//     device current).  Make that first call outside any stream capture.
#include "../../include/w4a16_b200.h"
#include "dec.h"

namespace {

constexpr size_t STATIC_PART_BYTES = 8u << 20;  // partial sums: 8 MiB = 1024 (split, row-block) pairs
constexpr size_t STATIC_TICKETS = 4096;         // arrival tickets (one unsigned per 256-row block)
constexpr size_t STATIC_BYTES = STATIC_TICKETS * sizeof(unsigned) + STATIC_PART_BYTES;

// In host code this name is only a handle for cudaGetSymbolAddress, never a device address.
static __device__ __align__(256) unsigned char g_static_scratch[STATIC_BYTES];

constexpr int MAX_DEVICES = 64;
unsigned char* g_scratch_addr[MAX_DEVICES] = {};

// Device address of the array on the CURRENT device (looked up once per device).
cudaError_t static_scratch(int device, unsigned char** out) {
    if (g_scratch_addr[device] == nullptr) {
        unsigned char* p = nullptr;
        cudaError_t e = cudaGetSymbolAddress((void**)&p, g_static_scratch);
        if (e != cudaSuccess) {
            return e;
        }
        g_scratch_addr[device] = p;
    }
    *out = g_scratch_addr[device];
    return cudaSuccess;
}

}  // namespace

extern "C" int w4a16_sk_single_static(w4a16_dec* dec, const char* name, const void* x16_dev, void* out_dev, int t,
                                      int out_kind, void* stream) {
    using namespace w4;
    Dec& d = dec->d;
    auto it = d.lins.find(name ? name : "");
    if (it == d.lins.end()) {
        return d.fail("w4a16: unknown linear %s", name ? name : "(null)");
    }
    const Lin& l = it->second;
    if (t < 1 || t > GEMV_MAX_M) {
        return d.fail("w4a16 sk_single_static: t=%d outside 1..%d", t, GEMV_MAX_M);
    }
    if (((uintptr_t)x16_dev & 15) != 0 || ((uintptr_t)out_dev & 15) != 0) {
        return d.fail("w4a16 sk_single_static: x and out must be 16-byte aligned");
    }
    int cur = -1;
    cudaError_t e = cudaGetDevice(&cur);
    if (e != cudaSuccess || cur != d.device || cur < 0 || cur >= MAX_DEVICES) {
        return d.fail("w4a16 sk_single_static: device %d must be current (current is %d)", d.device, cur);
    }
    unsigned char* base = nullptr;
    e = static_scratch(cur, &base);
    if (e != cudaSuccess) {
        return d.cuda_fail("cudaGetSymbolAddress(static scratch)", e);
    }

    GemvArgs a{};
    a.nseg = 1;
    a.k = l.k;
    a.group = l.group;
    a.seg[0].qt = (const uint4*)l.qt;
    a.seg[0].st = (const uint32_t*)l.st;
    a.seg[0].out = out_dev;
    a.seg[0].n = l.n;
    a.seg[0].out_mul = l.out_mul;
    a.m = t;
    a.out_f16 = out_kind == W4A16_OUT_F16;
    a.x = (const uint16_t*)x16_dev;
    cudaStream_t st = stream ? (cudaStream_t)stream : d.stream;
    // the same kernel form and plan as w4a16_sk_single_dev (shared selection), so the two give identical results
    GemvChoice c;
    if (int rc = d.gemv_select(a, false, true, c)) {
        return rc;
    }
    const size_t need = c.part_floats * sizeof(float);
    if (need > STATIC_PART_BYTES || c.tickets > STATIC_TICKETS) {
        return d.fail("w4a16 sk_single_static: %s needs %zu bytes of partial-sum scratch and %zu tickets; the built-in "
                      "array holds %zu bytes and %zu tickets (use w4a16_sk_single_dev)",
                      name, need, c.tickets, STATIC_PART_BYTES, STATIC_TICKETS);
    }
    a.pdl = 0;  // ordinary launch: the shared array must not be touched while an earlier kernel still runs
    a.dbg = nullptr;
    a.dbg_seq = 0;
    a.counters = reinterpret_cast<unsigned*>(base);
    a.part = reinterpret_cast<float*>(base + STATIC_TICKETS * sizeof(unsigned));
    // tickets must start at zero; the previous call may have been abandoned half-way
    e = cudaMemsetAsync(a.counters, 0, c.tickets * sizeof(unsigned), st);
    if (e != cudaSuccess) {
        return d.cuda_fail("clear tickets (static scratch)", e);
    }
    return d.gemv_run(a, c, st);
}
