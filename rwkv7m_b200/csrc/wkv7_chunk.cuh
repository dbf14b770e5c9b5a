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
