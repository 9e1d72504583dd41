// Optimizer-side flat kernels: AdamW on a contiguous shard and squared-norm accumulation.
//
// AdamW reads the gradient (fp32 or bf16), the fp32 master weights and the two
// moments (fp32 or bf16), applies the clip coefficient, decoupled weight decay and
// bias correction in fp32 and writes master, moments and the low-precision copy of
// the weights in one pass (7 streams through HBM instead of PyTorch's separate
// cast / clip / update / copy passes).  A non-finite clip coefficient means "skip
// this step": nothing is written.
#include <ATen/ATen.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>

#include "common.cuh"

namespace tb200 {

template <typename G, typename S, typename P>
__global__ void __launch_bounds__(256) adamw_kernel(float* __restrict__ master, const G* __restrict__ grad,
                                                    S* __restrict__ m, S* __restrict__ v, P* __restrict__ lowp,
                                                    const float* __restrict__ grad_scale, int64_t n, float lr,
                                                    float beta1, float beta2, float eps, float wd, float bc1,
                                                    float bc2_sqrt) {
  const float gs = *grad_scale;
  if (!isfinite(gs)) return;
  const float step_size = lr / bc1;
  const float decay = 1.f - lr * wd;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x * 4;
  for (int64_t base = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) * 4; base < n; base += stride) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int64_t i = base + j;
      if (i < n) {
        const float g = to_float<G>(grad[i]) * gs;
        float mm = to_float<S>(m[i]);
        float vv = to_float<S>(v[i]);
        mm = beta1 * mm + (1.f - beta1) * g;
        vv = beta2 * vv + (1.f - beta2) * g * g;
        float p = master[i] * decay;
        const float denom = sqrtf(vv) / bc2_sqrt + eps;
        p -= step_size * (mm / denom);
        master[i] = p;
        m[i] = from_float<S>(mm);
        v[i] = from_float<S>(vv);
        if (lowp != nullptr) lowp[i] = from_float<P>(p);
      }
    }
  }
}

// 8 elements per thread per iteration with 16-byte accesses (two for fp32 streams).
template <typename T>
__device__ __forceinline__ void load8(const T* p, float (&f)[8]);
template <>
__device__ __forceinline__ void load8<float>(const float* p, float (&f)[8]) {
  const float4 a = *reinterpret_cast<const float4*>(p);
  const float4 b = *reinterpret_cast<const float4*>(p + 4);
  f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
}
template <>
__device__ __forceinline__ void load8<__nv_bfloat16>(const __nv_bfloat16* p, float (&f)[8]) {
  unpack8(*reinterpret_cast<const bf16x8*>(p), f);
}
template <typename T>
__device__ __forceinline__ void store8(T* p, const float (&f)[8]);
template <>
__device__ __forceinline__ void store8<float>(float* p, const float (&f)[8]) {
  *reinterpret_cast<float4*>(p) = make_float4(f[0], f[1], f[2], f[3]);
  *reinterpret_cast<float4*>(p + 4) = make_float4(f[4], f[5], f[6], f[7]);
}
template <>
__device__ __forceinline__ void store8<__nv_bfloat16>(__nv_bfloat16* p, const float (&f)[8]) {
  *reinterpret_cast<bf16x8*>(p) = pack8(f);
}

template <typename G, typename S, typename P>
__global__ void __launch_bounds__(256) adamw_vec_kernel(float* __restrict__ master, const G* __restrict__ grad,
                                                        S* __restrict__ m, S* __restrict__ v, P* __restrict__ lowp,
                                                        const float* __restrict__ grad_scale, int64_t nvec, float lr,
                                                        float beta1, float beta2, float eps, float wd, float bc1,
                                                        float bc2_sqrt) {
  const float gs = *grad_scale;
  if (!isfinite(gs)) return;
  const float step_size = lr / bc1;
  const float decay = 1.f - lr * wd;
  const float inv_bc2 = 1.f / bc2_sqrt;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t o = i * 8;
    float g[8], mm[8], vv[8], p[8];
    load8<G>(grad + o, g);
    load8<S>(m + o, mm);
    load8<S>(v + o, vv);
    load8<float>(master + o, p);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float gj = g[j] * gs;
      mm[j] = beta1 * mm[j] + (1.f - beta1) * gj;
      vv[j] = beta2 * vv[j] + (1.f - beta2) * gj * gj;
      const float denom = sqrtf(vv[j]) * inv_bc2 + eps;
      p[j] = p[j] * decay - step_size * (mm[j] / denom);
    }
    store8<float>(master + o, p);
    store8<S>(m + o, mm);
    store8<S>(v + o, vv);
    if (lowp != nullptr) store8<P>(lowp + o, p);
  }
}


// 4 elements per access: a warp reads 512 contiguous bytes of every fp32 stream per instruction
// (each 32-byte sector is requested once), two independent groups per iteration for memory-level
// parallelism, streaming cache hints (nothing is reused).
template <typename T>
__device__ __forceinline__ void load4(const T* p, float (&f)[4]);
template <>
__device__ __forceinline__ void load4<float>(const float* p, float (&f)[4]) {
  const float4 a = __ldcs(reinterpret_cast<const float4*>(p));
  f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w;
}
template <>
__device__ __forceinline__ void load4<__nv_bfloat16>(const __nv_bfloat16* p, float (&f)[4]) {
  const uint2 a = __ldcs(reinterpret_cast<const uint2*>(p));
  const float2 lo = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&a.x));
  const float2 hi = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&a.y));
  f[0] = lo.x; f[1] = lo.y; f[2] = hi.x; f[3] = hi.y;
}
template <typename T>
__device__ __forceinline__ void store4(T* p, const float (&f)[4]);
template <>
__device__ __forceinline__ void store4<float>(float* p, const float (&f)[4]) {
  __stcs(reinterpret_cast<float4*>(p), make_float4(f[0], f[1], f[2], f[3]));
}
template <>
__device__ __forceinline__ void store4<__nv_bfloat16>(__nv_bfloat16* p, const float (&f)[4]) {
  __nv_bfloat162 lo = __floats2bfloat162_rn(f[0], f[1]), hi = __floats2bfloat162_rn(f[2], f[3]);
  uint2 w;
  w.x = *reinterpret_cast<uint32_t*>(&lo);
  w.y = *reinterpret_cast<uint32_t*>(&hi);
  *reinterpret_cast<uint2*>(p) = w;       // the low-precision weights are read by the next forward: default policy
}

template <typename G, typename S, typename P>
__global__ void __launch_bounds__(256) adamw_vec4_kernel(float* __restrict__ master, const G* __restrict__ grad,
                                                         S* __restrict__ m, S* __restrict__ v, P* __restrict__ lowp,
                                                         const float* __restrict__ grad_scale, int64_t nvec, float lr,
                                                         float beta1, float beta2, float eps, float wd, float bc1,
                                                         float bc2_sqrt) {
  const float gs = *grad_scale;
  if (!isfinite(gs)) return;
  const float step_size = lr / bc1;
  const float decay = 1.f - lr * wd;
  const float inv_bc2 = 1.f / bc2_sqrt;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i0 = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i0 < nvec; i0 += 2 * stride) {
    float g[2][4], mm[2][4], vv[2][4], p[2][4];
    bool live[2];
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      const int64_t o = (i0 + u * stride) * 4;
      live[u] = i0 + u * stride < nvec;
      if (live[u]) {
        load4<G>(grad + o, g[u]);
        load4<S>(m + o, mm[u]);
        load4<S>(v + o, vv[u]);
        load4<float>(master + o, p[u]);
      }
    }
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      if (!live[u]) continue;
      const int64_t o = (i0 + u * stride) * 4;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float gj = g[u][j] * gs;
        mm[u][j] = beta1 * mm[u][j] + (1.f - beta1) * gj;
        vv[u][j] = beta2 * vv[u][j] + (1.f - beta2) * gj * gj;
        const float denom = sqrtf(vv[u][j]) * inv_bc2 + eps;
        p[u][j] = p[u][j] * decay - step_size * (mm[u][j] / denom);
      }
      store4<float>(master + o, p[u]);
      store4<S>(m + o, mm[u]);
      store4<S>(v + o, vv[u]);
      if (lowp != nullptr) store4<P>(lowp + o, p[u]);
    }
  }
}

static inline bool is_aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

template <typename G, typename S, typename P>
static void launch_adamw(float* master, const G* grad, S* m, S* v, P* lowp, const float* gs, int64_t n, float lr,
                         float b1, float b2, float eps, float wd, float bc1, float bc2, cudaStream_t stream) {
  const int threads = 256;
  const bool vec = is_aligned16(master) && is_aligned16(grad) && is_aligned16(m) && is_aligned16(v) &&
                   (lowp == nullptr || is_aligned16(lowp));
  int64_t done = 0;
  if (vec && n >= 8) {
    const int64_t nvec = n / 4;
    const int grid = (int)std::max<int64_t>(1, std::min<int64_t>((nvec + 2 * threads - 1) / (2 * threads), (int64_t)num_sms() * 8));
    adamw_vec4_kernel<G, S, P><<<grid, threads, 0, stream>>>(master, grad, m, v, lowp, gs, nvec, lr, b1, b2, eps, wd,
                                                             bc1, sqrtf(bc2));
    done = nvec * 4;
  }
  if (done < n) {
    const int64_t rem = n - done;
    const int64_t want = (rem + threads * 4 - 1) / (threads * 4);
    const int grid = (int)std::max<int64_t>(1, std::min<int64_t>(want, (int64_t)num_sms() * 16));
    adamw_kernel<G, S, P><<<grid, threads, 0, stream>>>(master + done, grad + done, m + done, v + done,
                                                        lowp ? lowp + done : nullptr, gs, rem, lr, b1, b2, eps, wd, bc1,
                                                        sqrtf(bc2));
  }
}

void adamw_(at::Tensor master, const at::Tensor& grad, at::Tensor exp_avg, at::Tensor exp_avg_sq,
            const c10::optional<at::Tensor>& lowp, const at::Tensor& grad_scale, double lr, double beta1,
            double beta2, double eps, double weight_decay, double bc1, double bc2) {
  TORCH_CHECK(master.is_cuda() && master.scalar_type() == at::kFloat && master.is_contiguous());
  const int64_t n = master.numel();
  TORCH_CHECK(grad.numel() == n && exp_avg.numel() == n && exp_avg_sq.numel() == n);
  TORCH_CHECK(grad.is_contiguous() && exp_avg.is_contiguous() && exp_avg_sq.is_contiguous());
  TORCH_CHECK(exp_avg.scalar_type() == exp_avg_sq.scalar_type());
  TORCH_CHECK(grad_scale.scalar_type() == at::kFloat && grad_scale.numel() == 1 && grad_scale.is_cuda());
  if (lowp.has_value()) TORCH_CHECK(lowp->numel() == n && lowp->is_contiguous());
  if (n == 0) return;
  c10::cuda::CUDAGuard guard(master.device());
  auto stream = at::cuda::getCurrentCUDAStream();
  const auto gt = grad.scalar_type(), st = exp_avg.scalar_type();
  const auto pt = lowp.has_value() ? lowp->scalar_type() : at::kBFloat16;
  void* lp = lowp.has_value() ? lowp->data_ptr() : nullptr;
  const float* gs = grad_scale.data_ptr<float>();
  float* mp = master.data_ptr<float>();
#define TB_ADAMW(GT, ST, PT)                                                                              \
  launch_adamw<GT, ST, PT>(mp, reinterpret_cast<const GT*>(grad.data_ptr()),                               \
                           reinterpret_cast<ST*>(exp_avg.data_ptr()), reinterpret_cast<ST*>(exp_avg_sq.data_ptr()), \
                           reinterpret_cast<PT*>(lp), gs, n, (float)lr, (float)beta1, (float)beta2, (float)eps,    \
                           (float)weight_decay, (float)bc1, (float)bc2, stream)
  using bf16 = __nv_bfloat16;
  const bool gb = gt == at::kBFloat16, sb = st == at::kBFloat16, pb = pt == at::kBFloat16;
  TORCH_CHECK(gb || gt == at::kFloat, "adamw_: grad must be fp32 or bf16");
  TORCH_CHECK(sb || st == at::kFloat, "adamw_: moments must be fp32 or bf16");
  TORCH_CHECK(pb || pt == at::kFloat, "adamw_: low-precision copy must be fp32 or bf16");
  if (gb && sb && pb) TB_ADAMW(bf16, bf16, bf16);
  else if (gb && sb && !pb) TB_ADAMW(bf16, bf16, float);
  else if (gb && !sb && pb) TB_ADAMW(bf16, float, bf16);
  else if (gb && !sb && !pb) TB_ADAMW(bf16, float, float);
  else if (!gb && sb && pb) TB_ADAMW(float, bf16, bf16);
  else if (!gb && sb && !pb) TB_ADAMW(float, bf16, float);
  else if (!gb && !sb && pb) TB_ADAMW(float, float, bf16);
  else TB_ADAMW(float, float, float);
#undef TB_ADAMW
  C10_CUDA_KERNEL_LAUNCH_CHECK();
}

template <typename T>
__global__ void __launch_bounds__(256) sumsq_kernel(const T* __restrict__ x, float* __restrict__ acc, int64_t n,
                                                    int64_t nvec) {
  __shared__ float red[32];
  float s = 0.f;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += (int64_t)gridDim.x * blockDim.x) {
    float f[8];
    load8<T>(x + i * 8, f);
#pragma unroll
    for (int j = 0; j < 8; ++j) s += f[j] * f[j];
  }
  for (int64_t i = nvec * 8 + (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (int64_t)gridDim.x * blockDim.x) {
    const float f = to_float<T>(x[i]);
    s += f * f;
  }
  s = block_sum(s, red);
  if (threadIdx.x == 0) atomicAdd(acc, s);
}

void sumsq_(const at::Tensor& x, at::Tensor acc) {
  TORCH_CHECK(x.is_cuda() && x.is_contiguous() && acc.scalar_type() == at::kFloat && acc.numel() == 1);
  const int64_t n = x.numel();
  if (n == 0) return;
  c10::cuda::CUDAGuard guard(x.device());
  auto stream = at::cuda::getCurrentCUDAStream();
  const int64_t nvec = is_aligned16(x.data_ptr()) ? n / 8 : 0;
  const int grid = (int)std::max<int64_t>(1, std::min<int64_t>((n / 8 + 255) / 256 + 1, (int64_t)num_sms() * 8));
  if (x.scalar_type() == at::kFloat)
    sumsq_kernel<float><<<grid, 256, 0, stream>>>(x.data_ptr<float>(), acc.data_ptr<float>(), n, nvec);
  else if (x.scalar_type() == at::kBFloat16)
    sumsq_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>(reinterpret_cast<const __nv_bfloat16*>(x.data_ptr()),
                                                          acc.data_ptr<float>(), n, nvec);
  else
    TORCH_CHECK(false, "sumsq_: unsupported dtype");
  C10_CUDA_KERNEL_LAUNCH_CHECK();
}

}  // namespace tb200
