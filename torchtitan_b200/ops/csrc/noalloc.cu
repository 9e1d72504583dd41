// Allocation-free RMSNorm backward: see noalloc.h for the contract.
#include <cuda_runtime.h>

#include <atomic>
#include <mutex>

#include "common.cuh"
#include "noalloc.h"

namespace {

using namespace tb200;

// Partial weight-gradient sums, one row per thread group.  On the host this name is only
// a stand-in for the symbol; the device address comes from cudaGetSymbolAddress below.
static __device__ __align__(256) float g_partials[TB200_NOALLOC_MAX_GROUPS * TB200_NOALLOC_MAX_DIM];

template <typename T>
struct Vec;
template <>
struct Vec<__nv_bfloat16> {
  static constexpr int N = 8;
  static __device__ __forceinline__ void load(const __nv_bfloat16* p, float (&f)[8]) {
    unpack8(*reinterpret_cast<const bf16x8*>(p), f);
  }
  static __device__ __forceinline__ void store(__nv_bfloat16* p, const float (&f)[8]) {
    *reinterpret_cast<bf16x8*>(p) = pack8(f);
  }
};
template <>
struct Vec<float> {
  static constexpr int N = 4;
  static __device__ __forceinline__ void load(const float* p, float (&f)[4]) {
    const float4 v = *reinterpret_cast<const float4*>(p);
    f[0] = v.x; f[1] = v.y; f[2] = v.z; f[3] = v.w;
  }
  static __device__ __forceinline__ void store(float* p, const float (&f)[4]) {
    *reinterpret_cast<float4*>(p) = make_float4(f[0], f[1], f[2], f[3]);
  }
};

// One CTA per group; a group walks rows group, group + G, ...  Each thread owns up to VPT
// vectors of the row and keeps their weight-gradient partial sums in registers.
template <typename T, int VPT>
__global__ void __launch_bounds__(256) rmsnorm_bwd_static_kernel(const T* __restrict__ dy, const T* __restrict__ x,
                                                                 const T* __restrict__ w,
                                                                 const float* __restrict__ rstd_in, T* __restrict__ dx,
                                                                 float* __restrict__ partials, int64_t rows, int D) {
  constexpr int N = Vec<T>::N;
  __shared__ float red[32];
  const int nvec = D / N;
  float dwacc[VPT][N];
#pragma unroll
  for (int i = 0; i < VPT; ++i)
#pragma unroll
    for (int j = 0; j < N; ++j) dwacc[i][j] = 0.f;
  for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
    const float rstd = rstd_in[row];
    float xh[VPT][N], g[VPT][N];
    float dot = 0.f;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int v = threadIdx.x + i * blockDim.x;
      if (v < nvec) {
        float xf[N], df[N], wf[N];
        Vec<T>::load(x + row * D + v * N, xf);
        Vec<T>::load(dy + row * D + v * N, df);
        Vec<T>::load(w + v * N, wf);
#pragma unroll
        for (int j = 0; j < N; ++j) {
          xh[i][j] = xf[j] * rstd;
          dwacc[i][j] += df[j] * xh[i][j];
          g[i][j] = df[j] * wf[j];
          dot += g[i][j] * xh[i][j];
        }
      }
    }
    dot = block_sum(dot, red);
    const float c = dot / (float)D;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int v = threadIdx.x + i * blockDim.x;
      if (v < nvec) {
        float o[N];
#pragma unroll
        for (int j = 0; j < N; ++j) o[j] = (g[i][j] - xh[i][j] * c) * rstd;
        Vec<T>::store(dx + row * D + v * N, o);
      }
    }
  }
  // Every group writes its complete row of partials (zeros included), so the scratch needs no clearing.
  float* out = partials + (int64_t)blockIdx.x * D;
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int v = threadIdx.x + i * blockDim.x;
    if (v < nvec) {
#pragma unroll
      for (int j = 0; j < N; ++j) out[v * N + j] = dwacc[i][j];
    }
  }
}

__global__ void __launch_bounds__(256) reduce_partials_kernel(const float* __restrict__ partials,
                                                              float* __restrict__ dw, int groups, int D) {
  const int col = blockIdx.x * blockDim.x + threadIdx.x;
  if (col >= D) return;
  float s = 0.f;
  for (int p = 0; p < groups; ++p) s += partials[(int64_t)p * D + col];
  dw[col] = s;
}

constexpr int kMaxDevices = 64;
std::mutex g_mu;
float* g_scratch_ptr[kMaxDevices] = {nullptr};
std::atomic<int> g_last_cuda_error{0};   // written by any host thread, outside the set-up mutex too

// Device address of g_partials for the current device; looked up once per device.
int scratch_for_current_device(float** out) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
    g_last_cuda_error = (int)(e != cudaSuccess ? e : cudaErrorInvalidDevice);
    return TB200_NOALLOC_E_CUDA;
  }
  std::lock_guard<std::mutex> lock(g_mu);
  if (g_scratch_ptr[dev] == nullptr) {
    float* p = nullptr;
    e = cudaGetSymbolAddress((void**)&p, g_partials);
    if (e != cudaSuccess || p == nullptr) {
      g_last_cuda_error = (int)e;
      return TB200_NOALLOC_E_CUDA;
    }
    g_scratch_ptr[dev] = p;
  }
  *out = g_scratch_ptr[dev];
  return TB200_NOALLOC_OK;
}

inline bool aligned16(const void* p) { return p != nullptr && (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

template <typename T>
int launch(const void* dy, const void* x, const void* w, const float* rstd, void* dx, float* dw, int64_t rows, int D,
           float* scratch, cudaStream_t stream) {
  constexpr int N = Vec<T>::N;
  const int nvec = D / N;
  const int groups = (int)(rows < TB200_NOALLOC_MAX_GROUPS ? (rows > 0 ? rows : 1) : TB200_NOALLOC_MAX_GROUPS);
  const int vpt = nvec <= 256 ? 1 : (nvec <= 512 ? 2 : (nvec <= 1024 ? 4 : 8));
  int threads = (nvec + vpt - 1) / vpt;
  threads = (threads + 31) / 32 * 32;
  auto dyp = static_cast<const T*>(dy);
  auto xp = static_cast<const T*>(x);
  auto wp = static_cast<const T*>(w);
  auto dxp = static_cast<T*>(dx);
  switch (vpt) {
    case 1: rmsnorm_bwd_static_kernel<T, 1><<<groups, threads, 0, stream>>>(dyp, xp, wp, rstd, dxp, scratch, rows, D); break;
    case 2: rmsnorm_bwd_static_kernel<T, 2><<<groups, threads, 0, stream>>>(dyp, xp, wp, rstd, dxp, scratch, rows, D); break;
    case 4: rmsnorm_bwd_static_kernel<T, 4><<<groups, threads, 0, stream>>>(dyp, xp, wp, rstd, dxp, scratch, rows, D); break;
    default: rmsnorm_bwd_static_kernel<T, 8><<<groups, threads, 0, stream>>>(dyp, xp, wp, rstd, dxp, scratch, rows, D); break;
  }
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    g_last_cuda_error = (int)e;
    return TB200_NOALLOC_E_CUDA;
  }
  reduce_partials_kernel<<<(D + 255) / 256, 256, 0, stream>>>(scratch, dw, groups, D);
  e = cudaGetLastError();
  if (e != cudaSuccess) {
    g_last_cuda_error = (int)e;
    return TB200_NOALLOC_E_CUDA;
  }
  return TB200_NOALLOC_OK;
}

}  // namespace

extern "C" int tb200_rmsnorm_bwd_noalloc(const void* dy, const void* x, const void* weight, const float* rstd,
                                         void* dx, float* dw, int64_t rows, int dim, int dtype, void* stream) {
  if (dim > TB200_NOALLOC_MAX_DIM) return TB200_NOALLOC_E_TOO_LARGE;
  if (dtype != 0 && dtype != 1) return TB200_NOALLOC_E_BAD_SHAPE;
  const int vecw = dtype == 0 ? 8 : 4;
  if (dim <= 0 || dim % vecw != 0 || rows < 0) return TB200_NOALLOC_E_BAD_SHAPE;
  if (!aligned16(dy) || !aligned16(x) || !aligned16(weight) || !aligned16(dx) || rstd == nullptr || dw == nullptr)
    return TB200_NOALLOC_E_BAD_POINTER;
  float* scratch = nullptr;
  const int rc = scratch_for_current_device(&scratch);
  if (rc != TB200_NOALLOC_OK) return rc;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (dtype == 0) return launch<__nv_bfloat16>(dy, x, weight, rstd, dx, dw, rows, dim, scratch, s);
  return launch<float>(dy, x, weight, rstd, dx, dw, rows, dim, scratch, s);
}

extern "C" const char* tb200_noalloc_strerror(int code) {
  switch (code) {
    case TB200_NOALLOC_OK: return "ok";
    case TB200_NOALLOC_E_TOO_LARGE: return "row length exceeds TB200_NOALLOC_MAX_DIM (8192): the static scratch array cannot hold it";
    case TB200_NOALLOC_E_BAD_SHAPE: return "bad shape or dtype: dim must be a positive multiple of 8 (bf16) or 4 (fp32), rows >= 0, dtype 0 or 1";
    case TB200_NOALLOC_E_BAD_POINTER: return "null pointer, or dy/x/weight/dx not 16-byte aligned";
    case TB200_NOALLOC_E_CUDA: return "a CUDA call failed; see tb200_noalloc_last_cuda_error()";
    default: return "unknown error code";
  }
}

extern "C" int tb200_noalloc_last_cuda_error(void) { return g_last_cuda_error.load(); }
