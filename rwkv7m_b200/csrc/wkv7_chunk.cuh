// Helpers shared by the chunked WKV7 forward and backward kernels: the 128-byte-swizzled operand tile layout
// (rows of 64 bf16 = 128 bytes, 8-row atoms of 1024 bytes) and its UMMA descriptors.
#pragma once

#include "common.cuh"

namespace rk {
namespace chunk {

// byte offset of 16-byte piece c16 of row `row` in a [rows][128 B] tile with 128-byte swizzle
__device__ __forceinline__ uint32_t sw128(int row, int c16) {
  return (uint32_t)((row >> 3) * 1024 + (row & 7) * 128 + ((c16 ^ (row & 7)) << 4));
}

__device__ __forceinline__ uint4 pack8(const float (&x)[8]) {
  uint4 o;
  __nv_bfloat162 h;
  h = __floats2bfloat162_rn(x[0], x[1]); o.x = *reinterpret_cast<uint32_t*>(&h);
  h = __floats2bfloat162_rn(x[2], x[3]); o.y = *reinterpret_cast<uint32_t*>(&h);
  h = __floats2bfloat162_rn(x[4], x[5]); o.z = *reinterpret_cast<uint32_t*>(&h);
  h = __floats2bfloat162_rn(x[6], x[7]); o.w = *reinterpret_cast<uint32_t*>(&h);
  return o;
}
__device__ __forceinline__ void unpack8(const uint4& raw, float (&x)[8]) {
  const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w[i]));
    x[2 * i] = f.x; x[2 * i + 1] = f.y;
  }
}

__device__ __forceinline__ uint64_t desc_k(uint32_t addr) { return umma_smem_desc_sw128(addr, 16, 1024); }
__device__ __forceinline__ uint64_t desc_mn(uint32_t addr, uint32_t lbo) { return umma_smem_desc_sw128(addr, lbo, 1024); }

// 32 fp32 accumulator values of one row -> four swizzled 16-byte bf16 pieces (pieces p0..p0+3 of `row`).
// keep(s) decides which columns survive the triangular mask.
template <typename Keep>
__device__ __forceinline__ void store_masked_bf16(uint8_t* tile, int row, int p0, const uint32_t (&v)[32], int s0, Keep keep) {
#pragma unroll
  for (int p = 0; p < 4; ++p) {
    float x[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) x[j] = keep(s0 + 8 * p + j) ? __uint_as_float(v[8 * p + j]) : 0.f;
    *reinterpret_cast<uint4*>(tile + sw128(row, p0 + p)) = pack8(x);
  }
}


__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gsrc) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(smem_dst)), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() {
  asm volatile("cp.async.commit_group;" ::: "memory");
  asm volatile("cp.async.wait_group 0;" ::: "memory");
}

// ---- (I - A)^-1 for a strictly lower-triangular 64 x 64 matrix, blocked ------------------------------------------------
// The per-chunk triangular system (I - A_ab) U = Z is not solved by a 63-step substitution: the inverse itself is
// formed once per chunk and then applied by one tcgen05 product.  Blocks of 16: the four diagonal blocks are
// inverted independently in fp32 (one thread per column, 15 short steps), then [[X00, 0], [X10, X11]] with
// X10 = X11 A10 X00 gives the two 32 x 32 diagonal blocks, and the same formula once more the full inverse.  The
// four small block products run as warp-level tf32 MMAs (fp32 accumulation) on operands that stay in shared memory;
// the result is rounded to bf16 for the tcgen05 product anyway.
//
// F:     fp32 [64][kInvStride], F[t * kInvStride + s] = A[t][s] for s < t and 0 elsewhere.  Overwritten: on return it
//        holds the inverse (unit diagonal, zeros above it).
// work:  kInvWorkFloats floats of scratch.
// tile:  receives the inverse as bf16 in the 128-byte-swizzled [64][64] operand layout (row = t, column = s).
// Every thread of the CTA must call it (the barriers inside are CTA-wide); threads 0..255 do the work, any further
// warps only take part in the barriers.  It ends with every thread's stores issued but not yet fenced.
constexpr int kInvStride = 68;
constexpr int kInvTmStride = 40;   // row stride of the product scratch: 16-byte aligned rows, conflict-free B fragments
constexpr int kInvWorkFloats = 4 * 256 + 32 * kInvTmStride;

// One 16 x 8 output tile of C = A B on the tensor cores (tf32 inputs, fp32 accumulate), operands row-major fp32 in
// shared memory.  A points at the tile's first row, B at its first column; KSTEPS * 8 is the reduction length.
// Lane (g = lane / 4, t = lane % 4) returns C[g][2t], C[g][2t+1], C[g+8][2t], C[g+8][2t+1].
template <int KSTEPS>
__device__ __forceinline__ void mma_tile_tf32(const float* A, int lda, const float* B, int ldb, float (&c)[4], int lane) {
  const int g = lane >> 2, t = lane & 3;
  c[0] = c[1] = c[2] = c[3] = 0.f;
#pragma unroll
  for (int ks = 0; ks < KSTEPS; ++ks) {
    const int k0 = 8 * ks;
    const uint32_t a0 = __float_as_uint(A[g * lda + k0 + t]);
    const uint32_t a1 = __float_as_uint(A[(g + 8) * lda + k0 + t]);
    const uint32_t a2 = __float_as_uint(A[g * lda + k0 + t + 4]);
    const uint32_t a3 = __float_as_uint(A[(g + 8) * lda + k0 + t + 4]);
    const uint32_t b0 = __float_as_uint(B[(k0 + t) * ldb + g]);
    const uint32_t b1 = __float_as_uint(B[(k0 + t + 4) * ldb + g]);
    asm volatile(
        "mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
  }
}

__device__ __forceinline__ void unit_lower_inverse_64(float* F, float* work, uint8_t* tile, int tid) {
  float* D = work;            // [4][16][16]: inverses of the diagonal blocks, D[blk][r][j]
  float* Tm = work + 1024;    // products in flight: [2][16] rows at level 1, [32] rows at level 2, stride kInvTmStride
  const int warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t4 = lane & 3;
  if (tid < 64) {
    const int blk = tid >> 4, j = tid & 15;
    const float* Ab = F + (16 * blk) * kInvStride + 16 * blk;
    float x[16];
#pragma unroll
    for (int r = 0; r < 16; ++r) x[r] = r == j ? 1.f : 0.f;
#pragma unroll
    for (int s_ = 0; s_ < 15; ++s_) {
#pragma unroll
      for (int r = s_ + 1; r < 16; ++r) x[r] = fmaf(Ab[r * kInvStride + s_], x[s_], x[r]);
    }
#pragma unroll
    for (int r = 0; r < 16; ++r) D[blk * 256 + r * 16 + j] = x[r];
  }
  __syncthreads();
  const bool worker = tid < 256;
  if (!worker) {
    // no role at levels 1 and 2: fall through to the barriers
  } else if (warp < 4) {   // level 1a: Tm[p] = A(2p+1, 2p) X(2p, 2p), one 16 x 8 tile per warp
    const int p = warp >> 1, n0 = (warp & 1) * 8;
    float c[4];
    mma_tile_tf32<2>(F + (32 * p + 16) * kInvStride + 32 * p, kInvStride, D + (2 * p) * 256 + n0, 16, c, lane);
    float* dst = Tm + (16 * p) * kInvTmStride + n0 + 2 * t4;
    *reinterpret_cast<float2*>(dst + g * kInvTmStride) = make_float2(c[0], c[1]);
    *reinterpret_cast<float2*>(dst + (g + 8) * kInvTmStride) = make_float2(c[2], c[3]);
  } else {          // meanwhile the diagonal blocks of F receive their inverses: thread -> (block, row, 8 columns)
    const int e = tid - 128, cb = e >> 5, cr = (e >> 1) & 15, cc = (e & 1) * 8;
    const float4 d0 = *reinterpret_cast<const float4*>(D + cb * 256 + cr * 16 + cc);
    const float4 d1 = *reinterpret_cast<const float4*>(D + cb * 256 + cr * 16 + cc + 4);
    float* dst = F + (16 * cb + cr) * kInvStride + 16 * cb + cc;
    *reinterpret_cast<float4*>(dst) = d0;
    *reinterpret_cast<float4*>(dst + 4) = d1;
  }
  __syncthreads();
  if (warp < 4) {   // level 1b: X(2p+1, 2p) = X(2p+1, 2p+1) Tm[p], written over A(2p+1, 2p)
    const int p = warp >> 1, n0 = (warp & 1) * 8;
    float c[4];
    mma_tile_tf32<2>(D + (2 * p + 1) * 256, 16, Tm + (16 * p) * kInvTmStride + n0, kInvTmStride, c, lane);
    float* dst = F + (32 * p + 16) * kInvStride + 32 * p + n0 + 2 * t4;
    *reinterpret_cast<float2*>(dst + g * kInvStride) = make_float2(c[0], c[1]);
    *reinterpret_cast<float2*>(dst + (g + 8) * kInvStride) = make_float2(c[2], c[3]);
  }
  __syncthreads();
  const int m0 = ((warp >> 2) & 1) * 16, n0 = (warp & 3) * 8;   // level 2: 32 x 32 outputs, one 16 x 8 tile per warp
  if (worker) {   // level 2a: Tm = A(32:64, 0:32) X(0:32, 0:32)
    float c[4];
    mma_tile_tf32<4>(F + (32 + m0) * kInvStride, kInvStride, F + n0, kInvStride, c, lane);
    float* dst = Tm + m0 * kInvTmStride + n0 + 2 * t4;
    *reinterpret_cast<float2*>(dst + g * kInvTmStride) = make_float2(c[0], c[1]);
    *reinterpret_cast<float2*>(dst + (g + 8) * kInvTmStride) = make_float2(c[2], c[3]);
  }
  __syncthreads();
  if (worker) {   // level 2b: X(32:64, 0:32) = X(32:64, 32:64) Tm, written over A(32:64, 0:32)
    float c[4];
    mma_tile_tf32<4>(F + (32 + m0) * kInvStride + 32, kInvStride, Tm + n0, kInvTmStride, c, lane);
    float* dst = F + (32 + m0) * kInvStride + n0 + 2 * t4;
    *reinterpret_cast<float2*>(dst + g * kInvStride) = make_float2(c[0], c[1]);
    *reinterpret_cast<float2*>(dst + (g + 8) * kInvStride) = make_float2(c[2], c[3]);
  }
  __syncthreads();
  if (worker) {   // bf16 operand tile: thread -> (row tid >> 2, 16 columns)
    const int row = tid >> 2, q = tid & 3;
    const float* src = F + row * kInvStride + 16 * q;
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const float4 lo = *reinterpret_cast<const float4*>(src + 8 * h);
      const float4 hi = *reinterpret_cast<const float4*>(src + 8 * h + 4);
      const float x[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
      *reinterpret_cast<uint4*>(tile + sw128(row, 2 * q + h)) = pack8(x);
    }
  }
}

// 32 lanes x 32 consecutive fp32 columns of tensor memory, as floats
__device__ __forceinline__ void tmem_ld_f32(uint32_t taddr, float (&f)[32]) {
  uint32_t v[32];
  tmem_ld_32x32(taddr, v);
  tmem_ld_wait();
#pragma unroll
  for (int j = 0; j < 32; ++j) f[j] = __uint_as_float(v[j]);
}

}  // namespace chunk
}  // namespace rk
