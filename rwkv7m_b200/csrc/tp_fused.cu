// Tensor-parallel sequence collectives over NVLink symmetric memory, fused with their neighbours.
//
// The residual stream is sharded over time: rank r holds tokens [r*Tl, (r+1)*Tl) of every batch row.
//   tp_gather_seq          out[b, r*Tl + t, :] = x_r[b, t, :]          every rank reads its peers' slices with plain
//                                                                       16-byte peer loads (the all-gather)
//   tp_reduce_scatter_add  out[b, t, :] = residual[b, t, :] + sum_r partial_r[b, rank*Tl + t, :]
//                          the row-parallel GEMM wrote its partial [B, T, C] result straight into a symmetric
//                          buffer; the sum over ranks is one multimem.ld_reduce (bf16x2, fp32 accumulate, added
//                          inside the NVSwitch) per 16 bytes, or plain peer loads without multicast, and the
//                          residual add rides in the same kernel (reduce-scatter + residual in one pass)
//   tp_barrier             arrival counters in every peer's scratch words; bounded wait (about two seconds),
//                          reports through an error word
// Peers are reached with ld/st/red and multimem instructions only.  Buffers are used alternately (two per
// role), so one barrier before each consumer is enough: a rank can only be two collectives ahead of a peer
// after that peer has passed the barrier in between.
// The reference has no counterpart: XLA inserts all-reduce / all-to-all for its feature-sharded layout
// (src/rwkv7m/model/nnx_model.py:203-212).
#include "common.cuh"
#include "kernels.h"

namespace rk {

namespace {

__device__ __forceinline__ uint64_t gtimer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

constexpr int kTpAuxBarrier = 0;   // [kMaxRanks] arrival counters, slot p is written by rank p
constexpr int kTpAuxError = 16;    // non-zero after a wait ran out

__global__ void tp_barrier_kernel(TpPeers peers, uint32_t target) {
  const int p = threadIdx.x;
  if (p >= peers.world) return;
  uint32_t* my_aux = reinterpret_cast<uint32_t*>(peers.aux[peers.rank]);
  uint32_t* peer_aux = reinterpret_cast<uint32_t*>(peers.aux[p]);
  __threadfence_system();
  asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(peer_aux + kTpAuxBarrier + peers.rank), "r"(1u) : "memory");
  const uint32_t* mine = my_aux + kTpAuxBarrier + p;
  const uint64_t t0 = gtimer_ns();
  bool ok = false;
  for (uint32_t it = 0; it < (1u << 28); ++it) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(mine) : "memory");
    if (v >= target) { ok = true; break; }
    if ((it & 63u) == 63u && gtimer_ns() - t0 > 2000000000ull) break;
  }
  if (!ok) atomicExch(reinterpret_cast<int*>(my_aux + kTpAuxError), 0x50000 | p);
  __threadfence_system();
}

// grid: (pieces of one local slice row block, B, world); 16 bytes per thread per iteration
__global__ void __launch_bounds__(256) tp_gather_seq_kernel(TpPeers peers, __nv_bfloat16* __restrict__ out, int B, int Tl,
                                                            int C) {
  const int r = blockIdx.z, b = blockIdx.y;
  const uint4* src = reinterpret_cast<const uint4*>(peers.buf[r]) + (size_t)b * Tl * C / 8;
  uint4* dst = reinterpret_cast<uint4*>(out) + ((size_t)b * peers.world + r) * Tl * C / 8;
  const size_t n = (size_t)Tl * C / 8;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) dst[i] = src[i];
}

__device__ __forceinline__ void acc_bf16x8(float (&a)[8], const uint4& raw) {
  const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w[i]));
    a[2 * i] += f.x; a[2 * i + 1] += f.y;
  }
}

// grid: (blocks over one local slice, B)
template <bool MULTIMEM>
__global__ void __launch_bounds__(256) tp_reduce_scatter_add_kernel(TpPeers peers, const __nv_bfloat16* __restrict__ residual,
                                                                    __nv_bfloat16* __restrict__ out, int B, int Tl, int C) {
  const int b = blockIdx.y;
  const size_t n = (size_t)Tl * C / 8;                                                   // 16-byte pieces per (b, slice)
  const size_t src_off = ((size_t)b * peers.world + peers.rank) * Tl * C / 8;            // inside a full [B, T, C] buffer
  const size_t dst_off = (size_t)b * Tl * C / 8;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    float a[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) a[j] = 0.f;
    if (MULTIMEM) {
      uint4 v;
      asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
                   : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                   : "l"(reinterpret_cast<const uint4*>(peers.buf_mc) + src_off + i)
                   : "memory");
      acc_bf16x8(a, v);
    } else {
      for (int p = 0; p < peers.world; ++p) acc_bf16x8(a, reinterpret_cast<const uint4*>(peers.buf[p])[src_off + i]);
    }
    if (residual != nullptr) acc_bf16x8(a, reinterpret_cast<const uint4*>(residual)[dst_off + i]);
    uint4 o;
    __nv_bfloat162 h;
    h = __floats2bfloat162_rn(a[0], a[1]); o.x = *reinterpret_cast<uint32_t*>(&h);
    h = __floats2bfloat162_rn(a[2], a[3]); o.y = *reinterpret_cast<uint32_t*>(&h);
    h = __floats2bfloat162_rn(a[4], a[5]); o.z = *reinterpret_cast<uint32_t*>(&h);
    h = __floats2bfloat162_rn(a[6], a[7]); o.w = *reinterpret_cast<uint32_t*>(&h);
    reinterpret_cast<uint4*>(out)[dst_off + i] = o;
  }
}

int blocks_for(size_t pieces) {
  size_t want = (pieces + 255) / 256;
  if (want > 148 * 4) want = 148 * 4;
  return want < 1 ? 1 : (int)want;
}

}  // namespace

void tp_barrier(const TpPeers& peers, uint32_t target, cudaStream_t st) { tp_barrier_kernel<<<1, 32, 0, st>>>(peers, target); }

void tp_gather_seq(const TpPeers& peers, void* out, int B, int Tl, int C, cudaStream_t st) {
  const int bx = blocks_for((size_t)Tl * C / 8);
  dim3 grid(bx > 64 ? 64 : bx, B, peers.world);
  tp_gather_seq_kernel<<<grid, 256, 0, st>>>(peers, (__nv_bfloat16*)out, B, Tl, C);
}

void tp_reduce_scatter_add(const TpPeers& peers, const void* residual, void* out, int B, int Tl, int C, cudaStream_t st) {
  const int bx = blocks_for((size_t)Tl * C / 8);
  dim3 grid(bx > 128 ? 128 : bx, B);
  if (peers.buf_mc != nullptr)
    tp_reduce_scatter_add_kernel<true><<<grid, 256, 0, st>>>(peers, (const __nv_bfloat16*)residual, (__nv_bfloat16*)out, B, Tl, C);
  else
    tp_reduce_scatter_add_kernel<false><<<grid, 256, 0, st>>>(peers, (const __nv_bfloat16*)residual, (__nv_bfloat16*)out, B, Tl, C);
}

int tp_aux_error_word() { return kTpAuxError; }
int tp_aux_words() { return 32; }

}  // namespace rk
