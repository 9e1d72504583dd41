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

// 16-byte vector version for the common all-aligned case (fp32 state, bf16 grad or fp32 grad).
template <typename G, typename S, typename P>
static void launch_adamw(float* master, const G* grad, S* m, S* v, P* lowp, const float* gs, int64_t n, float lr,
                         float b1, float b2, float eps, float wd, float bc1, float bc2, cudaStream_t stream) {
  const int threads = 256;
  const int64_t want = (n + threads * 4 - 1) / (threads * 4);
  const int grid = (int)std::max<int64_t>(1, std::min<int64_t>(want, (int64_t)num_sms() * 16));
  adamw_kernel<G, S, P><<<grid, threads, 0, stream>>>(master, grad, m, v, lowp, gs, n, lr, b1, b2, eps, wd, bc1,
                                                      sqrtf(bc2));
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
__global__ void __launch_bounds__(256) sumsq_kernel(const T* __restrict__ x, float* __restrict__ acc, int64_t n) {
  __shared__ float red[32];
  float s = 0.f;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
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
  const int grid = (int)std::max<int64_t>(1, std::min<int64_t>((n + 255) / 256, (int64_t)num_sms() * 8));
  if (x.scalar_type() == at::kFloat)
    sumsq_kernel<float><<<grid, 256, 0, stream>>>(x.data_ptr<float>(), acc.data_ptr<float>(), n);
  else if (x.scalar_type() == at::kBFloat16)
    sumsq_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>(reinterpret_cast<const __nv_bfloat16*>(x.data_ptr()),
                                                          acc.data_ptr<float>(), n);
  else
    TORCH_CHECK(false, "sumsq_: unsupported dtype");
  C10_CUDA_KERNEL_LAUNCH_CHECK();
}

}  // namespace tb200
