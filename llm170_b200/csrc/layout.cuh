// Device-resident weight layout shared by the decode GEMV and the prefill GEMM ("T64").
//
// The boundary receives compressed-tensors `pack-quantized` weights: u32 [N][K/8], element i of
// a row is the nibble at bits 4*(i&7) of word i>>3 and stores q+8; f16 scales [N][K/group]
// (crates/core/src/w4a16.rs:124-175).  The reference re-tiles them for mma.sync m16n8k16 on the
// host (crates/core/src/marlin.rs:2-43, [K/16][N/64] tiles of 128 words).  This library keeps ONE
// device copy in a different tiling chosen for B200:
//
//   qt : u32 [K/64][N/16][32 lanes][4 words]            (512 B per 16-row x 64-k tile, k-block major)
//   st : f16 [N/16][K/group][8][2]                      (pair j = scales of rows j and j+8; group 128 or 32 --
//                                                        64-channel groups are stored as two groups of 32)
//
// Inside a tile, lane = 4*g + t (g = 0..7, t = 0..3) and word w = 2*p + h (p, h in {0,1}) hold
// rows r0 = 16*rb + g and r1 = r0 + 8 at k = 64*kb + 32*p + 8*t + 4*h + {0,1,2,3}:
//
//   nibble position : 0      4      1      5      2      6      3      7
//   element         : r0,k+0 r0,k+1 r1,k+0 r1,k+1 r0,k+2 r0,k+3 r1,k+2 r1,k+3
//
// so that (word & 0x000f000f), (word & 0x00f000f0), and the same two masks of (word >> 8) are,
// in that order, the four half2 registers a0..a3 of an m16n8k16 A fragment whose 16 rows are the
// tile's rows -- and, for the GEMM, one lane's 16 bytes expand to four whole 16-byte chunks
// (8 consecutive k of one row) of a 128B-swizzled K-major shared-memory operand.
// A warp reads a tile with one 128-bit load per lane, fully coalesced.  Tiles are ordered k-block
// major: the tiles of neighbouring row blocks at one k-block are contiguous, so a CTA that owns R
// row blocks fetches R*512 contiguous bytes per k-block with ONE bulk copy (8 KB for the GEMM's 256-row
// tile and for the GEMV's 256-row CTA), and the CTAs running at any moment sweep a narrow band of memory.
#pragma once
#include <cstddef>
#include <cstdint>

namespace w4 {

constexpr int TILE_ROWS = 16;
constexpr int TILE_K = 64;
constexpr int TILE_WORDS = 128;  // u32 per tile

// Shape contract of the tiled layout (the reference's Marlin path requires k%128==0 && n%64==0,
// crates/backend-gpu/src/rawcuda/w4a16_dec/kernels/marlin.rs:110; this layout is less strict).
__host__ __device__ inline bool shape_ok(int n, int k, int group) {
    return n > 0 && k > 0 && (group == 128 || group == 64 || group == 32) && n % TILE_ROWS == 0 &&
           k % TILE_K == 0 && k % group == 0;
}

// Gate|up interleaving of MoE expert matrices.  The boundary format stacks, per expert, `f` gate rows then `f` up
// rows.  With F = f/16 > 0 the resident layout alternates their 16-row blocks -- block 2j = gate rows 16j..16j+15,
// block 2j+1 = the up rows of the same outputs -- so that the CTA (and the warp, and the epilogue thread) that ends
// up with a gate value also holds its up value and can apply silu(gate)*up itself.  F = 0: no interleaving.
__host__ __device__ inline int glu_dest_rb(int src_rb, int F) {
    if (F <= 0) {
        return src_rb;
    }
    const int e = src_rb / (2 * F), b = src_rb - e * 2 * F;
    return e * 2 * F + (b < F ? 2 * b : 2 * (b - F) + 1);
}
__host__ __device__ inline int glu_src_rb(int dest_rb, int F) {
    if (F <= 0) {
        return dest_rb;
    }
    const int e = dest_rb / (2 * F), d = dest_rb - e * 2 * F;
    return e * 2 * F + ((d & 1) ? F + (d >> 1) : (d >> 1));
}

// Index of the packed word that holds element (row, kk), and the nibble position inside it.
__host__ __device__ inline size_t word_index(int row, int kk, int n_total, int* nib_pos) {
    const int rb = row / TILE_ROWS, rr = row % TILE_ROWS;
    const int g = rr & 7, hi_row = rr >> 3;
    const int kb = kk / TILE_K, kr = kk % TILE_K;
    const int p = kr >> 5, t = (kr >> 3) & 3, h = (kr >> 2) & 1, e = kr & 3;
    // e: 0 -> pos 0, 1 -> pos 4, 2 -> pos 2, 3 -> pos 6 ; rows r1 shift by one position
    const int base = ((e & 1) << 2) | (e & 2);
    *nib_pos = base + hi_row;
    const size_t tile = (size_t)kb * (size_t)(n_total / TILE_ROWS) + (size_t)rb;
    return tile * TILE_WORDS + (size_t)(4 * g + t) * 4 + (size_t)(2 * p + h);
}

}  // namespace w4
