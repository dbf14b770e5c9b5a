// Allocation-free LayerNorm backward: see noalloc.h for the contract.
#include "noalloc.h"

#include <cstdint>
#include <mutex>

#include "common.cuh"
#include "kernels.h"

namespace {

// Scratch for the [parts, C] partial sums of dw and db.  In host code this name is only a
// stand-in for the symbol; the device address is fetched with cudaGetSymbolAddress below.
static __device__ __align__(256) float g_ln_scratch[2 * RWKV7M_NOALLOC_MAX_PARTS * RWKV7M_NOALLOC_MAX_C];

constexpr int kMaxDevices = 64;
float* g_scratch_addr[kMaxDevices] = {nullptr};
std::mutex g_mu;

// Device address of the scratch array on the current device, looked up once per device.
int scratch_for_current_device(float** out) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return RWKV7M_NOALLOC_ERR_CUDA;
  if (dev < 0 || dev >= kMaxDevices) return RWKV7M_NOALLOC_ERR_CUDA;
  std::lock_guard<std::mutex> lock(g_mu);
  if (g_scratch_addr[dev] == nullptr) {
    float* ptr = nullptr;
    if (cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_ln_scratch) != cudaSuccess || ptr == nullptr)
      return RWKV7M_NOALLOC_ERR_CUDA;
    g_scratch_addr[dev] = ptr;
  }
  *out = g_scratch_addr[dev];
  return RWKV7M_NOALLOC_OK;
}

// out[c] = sum over parts of part[p][c]; every element of out is written, so nothing has to start at zero.
__global__ void sum_parts_kernel(const float* __restrict__ part, int parts, int C, float* __restrict__ out) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C) return;
  float acc = 0.f;
  for (int p = 0; p < parts; ++p) acc += part[(size_t)p * C + c];
  out[c] = acc;
}

}  // namespace

extern "C" int rwkv7m_layernorm_bwd_noalloc(const void* dy, const void* x, const float* w, const float* mean,
                                            const float* rstd, void* dx, float* dw, float* db, int M, int C,
                                            void* stream) {
  if (dy == nullptr || x == nullptr || w == nullptr || mean == nullptr || rstd == nullptr || dx == nullptr ||
      dw == nullptr || db == nullptr)
    return RWKV7M_NOALLOC_ERR_ARG;
  // the fused widths read and write dy, x and dx as 16-byte vectors; a misaligned row pointer would fault on the GPU
  auto misaligned = [](const void* p, uintptr_t a) { return (reinterpret_cast<uintptr_t>(p) & (a - 1)) != 0; };
  if (misaligned(dy, 16) || misaligned(x, 16) || misaligned(dx, 16) || misaligned(w, 4) || misaligned(mean, 4) ||
      misaligned(rstd, 4) || misaligned(dw, 4) || misaligned(db, 4))
    return RWKV7M_NOALLOC_ERR_ARG;
  if (M < 1 || C < 2 || (C & 1) || C > RWKV7M_NOALLOC_MAX_C) return RWKV7M_NOALLOC_ERR_SIZE;
  float* scratch = nullptr;
  const int rc = scratch_for_current_device(&scratch);
  if (rc != RWKV7M_NOALLOC_OK) return rc;
  int parts = M / 256;
  if (parts < 1) parts = 1;
  if (parts > RWKV7M_NOALLOC_MAX_PARTS) parts = RWKV7M_NOALLOC_MAX_PARTS;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  float* dw_part = scratch;
  float* db_part = scratch + (size_t)RWKV7M_NOALLOC_MAX_PARTS * RWKV7M_NOALLOC_MAX_C;
  // the partial-sum kernel writes every [part, c] entry it later reads, so stale contents are harmless
  rk::layernorm_bwd(dy, x, w, mean, rstd, dx, dw_part, db_part, parts, M, C, st);
  const int blocks = (C + 255) / 256;
  sum_parts_kernel<<<blocks, 256, 0, st>>>(dw_part, parts, C, dw);
  sum_parts_kernel<<<blocks, 256, 0, st>>>(db_part, parts, C, db);
  return cudaGetLastError() == cudaSuccess ? RWKV7M_NOALLOC_OK : RWKV7M_NOALLOC_ERR_CUDA;
}

extern "C" const char* rwkv7m_noalloc_strerror(int code) {
  switch (code) {
    case RWKV7M_NOALLOC_OK: return "ok";
    case RWKV7M_NOALLOC_ERR_SIZE: return "size outside the supported range (C even, 2 <= C <= 8192, M >= 1)";
    case RWKV7M_NOALLOC_ERR_CUDA: return "CUDA runtime call failed";
    case RWKV7M_NOALLOC_ERR_ARG:
      return "null or misaligned pointer argument (dy, x, dx: 16-byte aligned; fp32 arrays: 4-byte aligned)";
  }
  return "unknown code";
}
