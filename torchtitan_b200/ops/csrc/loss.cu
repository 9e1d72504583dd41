// Fused cross entropy on a chunk of logits: online log-sum-exp, per-row loss and
// in-place conversion of the logits into d(loss)/d(logits).
//
// One CTA per row.  Pass 1 reads the row once and keeps a running (max, sum) per
// thread (online softmax), pass 2 re-reads it (the row was just touched, so this
// mostly hits L2) and overwrites it with (softmax - onehot) * scale.  Rows whose
// label is the ignore index produce zero loss and zero gradient.
#include <ATen/ATen.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>

#include "common.cuh"

namespace tb200 {

constexpr int64_t kIgnoreIndex = -100;

__device__ __forceinline__ void online_merge(float& m, float& s, float m2, float s2) {
  const float mm = fmaxf(m, m2);
  if (mm == -INFINITY) {
    m = mm;
    s = 0.f;
    return;
  }
  s = s * __expf(m - mm) + s2 * __expf(m2 - mm);
  m = mm;
}

template <typename T, int VEC>
__global__ void __launch_bounds__(1024) cross_entropy_kernel(T* __restrict__ logits, const int64_t* __restrict__ labels,
                                                             const float* __restrict__ scale_ptr,
                                                             float* __restrict__ row_loss, int V) {
  __shared__ float red_m[32];
  __shared__ float red_s[32];
  __shared__ float sh_lse;
  const int64_t row = blockIdx.x;
  T* lr = logits + row * (int64_t)V;
  const int64_t label = labels[row];
  const bool valid = label != kIgnoreIndex && label >= 0 && label < V;
  const float scale = valid ? *scale_ptr : 0.f;

  float m = -INFINITY, s = 0.f;
  if (VEC == 8) {
    const int nvec = V / 8;
    for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
      bf16x8 p = *reinterpret_cast<const bf16x8*>(reinterpret_cast<const __nv_bfloat16*>(lr) + v * 8);
      float f[8];
      unpack8(p, f);
      float lm = f[0];
#pragma unroll
      for (int j = 1; j < 8; ++j) lm = fmaxf(lm, f[j]);
      const float mm = fmaxf(m, lm);
      float acc = 0.f;
#pragma unroll
      for (int j = 0; j < 8; ++j) acc += __expf(f[j] - mm);
      s = s * __expf(m - mm) + acc;
      m = mm;
    }
  } else {
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
      const float x = to_float<T>(lr[i]);
      const float mm = fmaxf(m, x);
      s = s * __expf(m - mm) + __expf(x - mm);
      m = mm;
    }
  }
  // warp then block merge of (m, s)
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float m2 = __shfl_xor_sync(0xffffffffu, m, o);
    const float s2 = __shfl_xor_sync(0xffffffffu, s, o);
    online_merge(m, s, m2, s2);
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
  if (lane == 0) {
    red_m[warp] = m;
    red_s[warp] = s;
  }
  __syncthreads();
  if (warp == 0) {
    m = lane < nwarp ? red_m[lane] : -INFINITY;
    s = lane < nwarp ? red_s[lane] : 0.f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float m2 = __shfl_xor_sync(0xffffffffu, m, o);
      const float s2 = __shfl_xor_sync(0xffffffffu, s, o);
      online_merge(m, s, m2, s2);
    }
    if (lane == 0) {
      const float lse = m + __logf(s);
      sh_lse = lse;
      float loss = 0.f;
      if (valid) loss = lse - to_float<T>(lr[label]);
      row_loss[row] = loss;
    }
  }
  __syncthreads();
  const float lse = sh_lse;
  if (VEC == 8) {
    const int nvec = V / 8;
    const int lv = valid ? (int)(label / 8) : -1;
    const int lj = valid ? (int)(label % 8) : -1;
    for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
      __nv_bfloat16* ptr = reinterpret_cast<__nv_bfloat16*>(lr) + v * 8;
      bf16x8 p = *reinterpret_cast<const bf16x8*>(ptr);
      float f[8];
      unpack8(p, f);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        float g = __expf(f[j] - lse);
        if (v == lv && j == lj) g -= 1.f;
        f[j] = g * scale;
      }
      *reinterpret_cast<bf16x8*>(ptr) = pack8(f);
    }
  } else {
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
      float g = __expf(to_float<T>(lr[i]) - lse);
      if (valid && i == label) g -= 1.f;
      lr[i] = from_float<T>(g * scale);
    }
  }
}

// logits[T, V] -> dlogits in place; returns per-row losses [T] (fp32).
at::Tensor cross_entropy_(at::Tensor logits, const at::Tensor& labels, const at::Tensor& scale) {
  TORCH_CHECK(logits.is_cuda() && logits.dim() == 2 && logits.is_contiguous());
  TORCH_CHECK(labels.scalar_type() == at::kLong && labels.is_contiguous() && labels.numel() == logits.size(0));
  TORCH_CHECK(scale.scalar_type() == at::kFloat && scale.numel() == 1 && scale.is_cuda());
  const int64_t rows = logits.size(0);
  const int V = (int)logits.size(1);
  c10::cuda::CUDAGuard guard(logits.device());
  auto row_loss = at::empty({rows}, logits.options().dtype(at::kFloat));
  if (rows == 0) return row_loss;
  auto stream = at::cuda::getCurrentCUDAStream();
  int threads = 1024;
  while (threads > 64 && threads * 8 > V) threads /= 2;
  if (logits.scalar_type() == at::kBFloat16) {
    auto p = reinterpret_cast<__nv_bfloat16*>(logits.data_ptr());
    const bool vec = (V % 8 == 0) && (reinterpret_cast<uintptr_t>(p) % 16 == 0);
    if (vec)
      cross_entropy_kernel<__nv_bfloat16, 8><<<(unsigned)rows, threads, 0, stream>>>(
          p, labels.data_ptr<int64_t>(), scale.data_ptr<float>(), row_loss.data_ptr<float>(), V);
    else
      cross_entropy_kernel<__nv_bfloat16, 1><<<(unsigned)rows, threads, 0, stream>>>(
          p, labels.data_ptr<int64_t>(), scale.data_ptr<float>(), row_loss.data_ptr<float>(), V);
  } else if (logits.scalar_type() == at::kFloat) {
    cross_entropy_kernel<float, 1><<<(unsigned)rows, threads, 0, stream>>>(
        logits.data_ptr<float>(), labels.data_ptr<int64_t>(), scale.data_ptr<float>(), row_loss.data_ptr<float>(), V);
  } else {
    TORCH_CHECK(false, "cross_entropy_: unsupported dtype");
  }
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  return row_loss;
}

}  // namespace tb200
