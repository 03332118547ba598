// Shared device helpers and the tiled weight format of the MoE kernels.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace neon {

// ---------------------------------------------------------------------------------------
// Tiled MXFP4 weight format ("mma16" format), produced once by repack kernels.
//
// A row tile is 16 matrix rows, matching the M=16 of mma.m16n8k16.  MMA row g (0..7) and
// row g+8 are held by the same thread, so for gate_up the tile covers 8 intermediate
// channels: MMA row g = gate row 2*(8*tile+g), MMA row g+8 = linear row 2*(8*tile+g)+1;
// SwiGLU then needs no cross-thread traffic.  For down, MMA row r = matrix row 16*tile+r.
//
// K is walked in "block pairs" of 64 columns (two 32-wide MXFP4 scale blocks).  For tile
// `tl`, block pair `bp`, lane (g = lane/4, t = lane%4) the format stores one uint4:
//   .x = row g,   block 2bp    .y = row g+8, block 2bp
//   .z = row g,   block 2bp+1  .w = row g+8, block 2bp+1
// each word holding the 8 codes of columns 32*block + 8t + j, j = 0..7, bit-scattered so
// that bf16 pairs fall out with shifts and masks only (see pack8 / unpack below).
// Scales: one uint32 per (tile, block pair, g): bytes = (row g, blk 2bp), (row g+8, blk 2bp),
// (row g, blk 2bp+1), (row g+8, blk 2bp+1), each stored as (E8M0 byte + 126), the bf16
// exponent field of 2^(byte-1); E8M0 bytes 0..128 (scales up to 2) are representable.
// ---------------------------------------------------------------------------------------

// Scatter 8 e2m1 codes (c[j] = s e e m) into one word.  Pair q = (c[2q], c[2q+1]); the
// second element of a pair sits 16 bits above the first.  Per 16-bit half:
//   q=0: sign 15, magnitude 8..6     q=1: sign 12, magnitude 5..3
//   q=2: sign 14, magnitude 2..0     q=3: sign 13, magnitude 11..9
__host__ __device__ inline uint32_t pack8(const uint32_t c[8]) {
    const int sign_pos[4] = {15, 12, 14, 13};
    const int mag_pos[4] = {6, 3, 0, 9};
    uint32_t w = 0;
    for (int q = 0; q < 4; ++q)
        for (int hf = 0; hf < 2; ++hf) {
            uint32_t code = c[2 * q + hf] & 15u;
            w |= ((code >> 3) & 1u) << (sign_pos[q] + 16 * hf);
            w |= (code & 7u) << (mag_pos[q] + 16 * hf);
        }
    return w;
}

__device__ __forceinline__ uint32_t mul_bf16x2(uint32_t a, uint32_t b) {
    uint32_t d;
    asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
    return d;
}

// Placing s at bit 15 and e e m at bits 8..6 of a bf16 yields value * 2^-126 (the e2m1
// subnormal 0.5 becomes the bf16 subnormal 2^-127).  One multiply by 2^(126 + scale_exp)
// restores the value and applies the block scale exactly (powers of two only).
// `mult` = bf16x2 holding 2^(byte-1), i.e. exponent field (byte + 126), in both halves.
__device__ __forceinline__ void unpack8(uint32_t w, uint32_t mult, uint32_t out[4]) {
    const uint32_t M = 0x81C081C0u, MM = 0x01C001C0u, SM = 0x80008000u;
    uint32_t p0 = w & M;
    uint32_t p1 = (w << 3) & M;
    uint32_t p2 = ((w << 6) & MM) | ((w << 1) & SM);
    uint32_t p3 = ((w >> 3) & MM) | ((w << 2) & SM);
    out[0] = mul_bf16x2(p0, mult);
    out[1] = mul_bf16x2(p1, mult);
    out[2] = mul_bf16x2(p2, mult);
    out[3] = mul_bf16x2(p3, mult);
}

// Stored scale byte (E8M0 + 126) -> bf16x2 multiplier with that exponent field in both halves.
__device__ __forceinline__ uint32_t scale_mult(uint32_t field) { return field * 0x00800080u; }

__device__ __forceinline__ void mma_bf16_16816(float c[4], const uint32_t a[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// Programmatic dependent launch: a kernel launched with the programmatic-serialization attribute
// may start while its predecessor in the stream is still draining; pdl_wait() blocks until the
// predecessor has completed and its writes are visible, pdl_launch_dependents() lets the
// successor start launching.  Both are no-ops for ordinary launches.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

__device__ __forceinline__ float bf16_bits_to_float(uint16_t b) { return __uint_as_float((uint32_t)b << 16); }

__device__ __forceinline__ uint4 ldg_stream(const uint4* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}

}  // namespace neon
