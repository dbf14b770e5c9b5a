// Data-parallel optimizer step over NVLink symmetric memory.
//
// Every rank holds the full flat fp32 gradient buffer, the full fp32 master parameters and the
// bf16 compute copy in buffers that are mapped into all peers (and, when NVSwitch multicast is
// available, bound to one multicast address).  Rank r owns elements [r*S, (r+1)*S) of the Adam
// moments.  One optimizer step is
//
//   barrier            all ranks finished backward
//   reduce_shard       owned gradient shard = sum over ranks, read either with one
//                      multimem.ld_reduce per 16 bytes (the switch adds the replicas) or with
//                      plain peer loads; the sum of squares of the shard is accumulated
//   publish + barrier  every rank stores its partial sum of squares into each peer's slot
//   adamw_allgather    global-norm clip, AdamW on the owned shard, and the new fp32 master value
//                      plus its bf16 cast are stored to every rank (multimem.st or peer stores):
//                      the parameter all-gather is the epilogue of the optimizer kernel
//   barrier            new parameters have landed everywhere
//
// Peers are reached with plain ld/st/red and multimem instructions only.
// Every wait is bounded (two seconds unless dp_set_wait_limit_ms() says otherwise) and reports through an error
// word instead of hanging; once the word is set, the reduce and AdamW kernels of the same and of later steps
// return without touching memory, so a wait that ran out makes the step a no-op rather than a wrong update.
// The reference has no counterpart: its data parallelism is an XLA-inserted all-reduce with
// replicated optimizer state (src/rwkv7m/distributed/trainer.py:31-51).
#include "common.cuh"
#include "kernels.h"

namespace rk {

namespace {

__device__ __forceinline__ uint64_t gtimer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

__device__ __forceinline__ void red_release_sys_add(uint32_t* addr, uint32_t v) {
  asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(addr), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* addr) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(addr) : "memory");
  return v;
}
__device__ __forceinline__ void st_relaxed_sys_f32(float* addr, float v) {
  asm volatile("st.relaxed.sys.global.f32 [%0], %1;" ::"l"(addr), "f"(v) : "memory");
}

__device__ __forceinline__ float4 multimem_ld_reduce_f32x4(const float* mc_addr) {
  float4 r;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(r.x), "=f"(r.y), "=f"(r.z), "=f"(r.w)
               : "l"(mc_addr)
               : "memory");
  return r;
}
__device__ __forceinline__ void multimem_st_f32x4(float* mc_addr, float4 v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(mc_addr), "f"(v.x), "f"(v.y),
               "f"(v.z), "f"(v.w)
               : "memory");
}
__device__ __forceinline__ void multimem_st_b32x2(void* mc_addr, uint32_t a, uint32_t b) {
  asm volatile("multimem.st.relaxed.sys.global.v2.bf16x2 [%0], {%1, %2};" ::"l"(mc_addr), "r"(a), "r"(b) : "memory");
}

// aux word layout (uint32 / float words of the per-rank symmetric scratch buffer)
constexpr int kAuxBarrier = 0;    // [kMaxRanks] arrival counters, slot p is written by rank p
constexpr int kAuxNorm = 16;      // [2][kMaxRanks] partial sums of squares, double-buffered by step parity
constexpr int kAuxError = 48;     // non-zero after a wait ran out
constexpr int kAuxLocalNorm = 49; // this rank's partial sum of squares of the current step

uint64_t g_wait_limit_ns = 2000000000ull;   // host copy, passed to every barrier launch

__device__ __forceinline__ bool dp_failed(const DpPeers& peers, int rank) {
  return *reinterpret_cast<volatile const int*>(reinterpret_cast<const uint32_t*>(peers.aux[rank]) + kAuxError) != 0;
}

// One CTA, one thread per peer.  Optionally publishes this rank's partial norm first.
__global__ void dp_barrier_kernel(DpPeers peers, int rank, int world, uint32_t target, int publish_parity,
                                  uint64_t limit_ns) {
  const int p = threadIdx.x;
  if (p >= world) return;
  uint32_t* my_aux = reinterpret_cast<uint32_t*>(peers.aux[rank]);
  uint32_t* peer_aux = reinterpret_cast<uint32_t*>(peers.aux[p]);
  if (publish_parity >= 0) {
    const float part = reinterpret_cast<float*>(my_aux)[kAuxLocalNorm];
    st_relaxed_sys_f32(reinterpret_cast<float*>(peer_aux) + kAuxNorm + publish_parity * kMaxRanks + rank, part);
  }
  __threadfence_system();
  red_release_sys_add(peer_aux + kAuxBarrier + rank, 1u);
  const uint32_t* mine = my_aux + kAuxBarrier + p;
  const uint64_t t0 = gtimer_ns();
  bool ok = false;
  for (uint32_t it = 0; it < (1u << 28); ++it) {
    if (ld_acquire_sys(mine) >= target) { ok = true; break; }
    if ((it & 63u) == 63u && gtimer_ns() - t0 > limit_ns) break;
  }
  if (!ok) atomicExch(reinterpret_cast<int*>(my_aux + kAuxError), 0x20000 | p);
  __threadfence_system();
}

template <bool MULTIMEM>
__global__ void __launch_bounds__(256) dp_reduce_shard_kernel(DpPeers peers, int rank, int world, int64_t begin,
                                                              int64_t end) {
  if (dp_failed(peers, rank)) return;   // a barrier gave up: the peers' gradients may be unfinished
  float* my_grad = reinterpret_cast<float*>(peers.grad[rank]);
  float acc = 0.f;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x * 4;
  for (int64_t i = begin + ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) * 4; i < end; i += stride) {
    float4 g;
    if (MULTIMEM) {
      g = multimem_ld_reduce_f32x4(reinterpret_cast<const float*>(peers.grad_mc) + i);
    } else {
      g = make_float4(0.f, 0.f, 0.f, 0.f);
      for (int p = 0; p < world; ++p) {
        const float4 t = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(peers.grad[p]) + i);
        g.x += t.x; g.y += t.y; g.z += t.z; g.w += t.w;
      }
    }
    *reinterpret_cast<float4*>(my_grad + i) = g;
    acc += g.x * g.x + g.y * g.y + g.z * g.z + g.w * g.w;
  }
  acc = warp_sum(acc);
  __shared__ float part[8];
  if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x < 32) {
    float t = threadIdx.x < 8 ? part[threadIdx.x] : 0.f;
    t = warp_sum(t);
    if (threadIdx.x == 0) atomicAdd(reinterpret_cast<float*>(peers.aux[rank]) + kAuxLocalNorm, t);
  }
}

template <bool MULTIMEM>
__global__ void __launch_bounds__(256) dp_adamw_allgather_kernel(DpPeers peers, DpAdamW a) {
  if (dp_failed(peers, a.rank)) return;   // no update from partial sums
  const float* my_grad = reinterpret_cast<const float*>(peers.grad[a.rank]);
  float* my_master = reinterpret_cast<float*>(peers.master[a.rank]);
  const float* slots = reinterpret_cast<const float*>(peers.aux[a.rank]) + kAuxNorm + a.parity * kMaxRanks;
  float nsq = 0.f;
  for (int p = 0; p < a.world; ++p) nsq += slots[p];
  const float norm = sqrtf(nsq);
  const float clip = norm < a.max_norm ? 1.0f : a.max_norm / norm;
  if (blockIdx.x == 0 && threadIdx.x == 0) *a.norm_out = norm;
  const float inv_bc1 = 1.0f / a.bc1, inv_bc2 = 1.0f / a.bc2;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x * 4;
  for (int64_t i = a.begin + ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) * 4; i < a.end; i += stride) {
    const float4 g4 = *reinterpret_cast<const float4*>(my_grad + i);
    const float4 w4 = *reinterpret_cast<const float4*>(my_master + i);
    const int64_t li = i - a.begin;
    float4 m4 = *reinterpret_cast<const float4*>(a.m + li);
    float4 v4 = *reinterpret_cast<const float4*>(a.v + li);
    const float g[4] = {g4.x * clip, g4.y * clip, g4.z * clip, g4.w * clip};
    float w[4] = {w4.x, w4.y, w4.z, w4.w};
    float m[4] = {m4.x, m4.y, m4.z, m4.w};
    float v[4] = {v4.x, v4.y, v4.z, v4.w};
    const bool decay = i < a.n_decay;
    const float mult = i >= a.n_nodecay_end ? 2.0f : 1.0f;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      m[j] = a.beta1 * m[j] + (1.0f - a.beta1) * g[j];
      v[j] = a.beta2 * v[j] + (1.0f - a.beta2) * g[j] * g[j];
      float upd = (m[j] * inv_bc1) / (sqrtf(v[j] * inv_bc2) + a.eps);
      if (decay) upd += a.weight_decay * w[j];
      w[j] -= a.lr * mult * upd;
    }
    *reinterpret_cast<float4*>(a.m + li) = make_float4(m[0], m[1], m[2], m[3]);
    *reinterpret_cast<float4*>(a.v + li) = make_float4(v[0], v[1], v[2], v[3]);
    const float4 wn = make_float4(w[0], w[1], w[2], w[3]);
    const __nv_bfloat162 h0 = __floats2bfloat162_rn(w[0], w[1]);
    const __nv_bfloat162 h1 = __floats2bfloat162_rn(w[2], w[3]);
    const uint32_t b0 = *reinterpret_cast<const uint32_t*>(&h0), b1 = *reinterpret_cast<const uint32_t*>(&h1);
    const bool bcast_master = i >= a.master_bcast_from;
    if (!bcast_master) *reinterpret_cast<float4*>(my_master + i) = wn;
    if (MULTIMEM) {
      if (bcast_master) multimem_st_f32x4(reinterpret_cast<float*>(peers.master_mc) + i, wn);
      if (peers.shadow_mc != nullptr)
        multimem_st_b32x2(reinterpret_cast<__nv_bfloat16*>(peers.shadow_mc) + i, b0, b1);
    } else {
      for (int p = 0; p < a.world; ++p) {
        if (bcast_master) *reinterpret_cast<float4*>(reinterpret_cast<float*>(peers.master[p]) + i) = wn;
        if (peers.shadow[p] != nullptr)
          *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(peers.shadow[p]) + i) = make_uint2(b0, b1);
      }
    }
  }
}

int grid_for(int64_t n) {
  int64_t want = (n / 4 + 255) / 256;
  if (want > 148 * 8) want = 148 * 8;
  if (want < 1) want = 1;
  return (int)want;
}

}  // namespace

void dp_barrier(const DpPeers& peers, int rank, int world, uint32_t target, int publish_parity, cudaStream_t st) {
  dp_barrier_kernel<<<1, 32, 0, st>>>(peers, rank, world, target, publish_parity, g_wait_limit_ns);
}

void dp_set_wait_limit_ms(double ms) {
  if (ms < 1.0) ms = 1.0;
  g_wait_limit_ns = (uint64_t)(ms * 1.0e6);
}
double dp_wait_limit_ms() { return (double)g_wait_limit_ns / 1.0e6; }

void dp_reduce_shard(const DpPeers& peers, int rank, int world, int64_t begin, int64_t end, cudaStream_t st) {
  float* local = reinterpret_cast<float*>(peers.aux[rank]) + kAuxLocalNorm;
  cudaMemsetAsync(local, 0, sizeof(float), st);
  if (end <= begin) return;
  if (peers.grad_mc != nullptr)
    dp_reduce_shard_kernel<true><<<grid_for(end - begin), 256, 0, st>>>(peers, rank, world, begin, end);
  else
    dp_reduce_shard_kernel<false><<<grid_for(end - begin), 256, 0, st>>>(peers, rank, world, begin, end);
}

void dp_adamw_allgather(const DpPeers& peers, const DpAdamW& a, cudaStream_t st) {
  if (a.end <= a.begin) return;
  if (peers.master_mc != nullptr)
    dp_adamw_allgather_kernel<true><<<grid_for(a.end - a.begin), 256, 0, st>>>(peers, a);
  else
    dp_adamw_allgather_kernel<false><<<grid_for(a.end - a.begin), 256, 0, st>>>(peers, a);
}

int dp_aux_error_word() { return kAuxError; }
int dp_aux_words() { return 64; }

}  // namespace rk
