// Depthwise causal convolution over tokens followed by SiLU (the short convolution in front of the gated
// delta rule of Qwen3.5 / Qwen3-Next), forward and backward, for the folded-token layout x[T, C].
//
//   y[t, c] = silu( sum_{j < W} w[c, W-1-j] * x[t-j, c] * [pos[t] >= j] )
//
// `pos[t]` is the token's position inside its document, so a tap never reaches across a document boundary (without
// `pos` the whole tensor is one document).  One thread owns a group of 8 (bf16) or 4 (fp32) channels and a block of
// kRows consecutive tokens; it walks down the tokens with the last W-1 rows in registers, so x is read once
// (+ (W-1)/kRows halo) instead of W times.  The backward recomputes the pre-activation, forms
// ds = dy * silu'(pre), and produces dx (the transposed convolution of ds) and per-row-block partial sums of
// dw, which the host sums (deterministic).
#include <ATen/ATen.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/library.h>

#include "common.cuh"

namespace tb200 {
namespace {

constexpr int kRows = 64;      // tokens per thread
constexpr int kThreads = 128;  // channel groups per block
constexpr int kMaxW = 4;

template <typename T>
struct ChanVec;
template <>
struct ChanVec<__nv_bfloat16> {
  static constexpr int N = 8;
  static __device__ __forceinline__ void load(const __nv_bfloat16* p, float (&f)[8]) {
    unpack8(*reinterpret_cast<const bf16x8*>(p), f);
  }
  static __device__ __forceinline__ void store(__nv_bfloat16* p, const float (&f)[8]) {
    *reinterpret_cast<bf16x8*>(p) = pack8(f);
  }
};
template <>
struct ChanVec<float> {
  static constexpr int N = 4;
  static __device__ __forceinline__ void load(const float* p, float (&f)[4]) {
    const float4 v = *reinterpret_cast<const float4*>(p);
    f[0] = v.x; f[1] = v.y; f[2] = v.z; f[3] = v.w;
  }
  static __device__ __forceinline__ void store(float* p, const float (&f)[4]) {
    *reinterpret_cast<float4*>(p) = make_float4(f[0], f[1], f[2], f[3]);
  }
};

template <typename T, int W>
__global__ void __launch_bounds__(kThreads)
conv_silu_fwd_kernel(const T* __restrict__ x, const float* __restrict__ w, const int64_t* __restrict__ pos,
                     T* __restrict__ y, int64_t T_, int C) {
  using V = ChanVec<T>;
  constexpr int N = V::N;
  const int cg = blockIdx.x * kThreads + threadIdx.x;
  if (cg * N >= C) return;
  const int c0 = cg * N;
  const int64_t t0 = (int64_t)blockIdx.y * kRows;
  float wr[W][N];   // wr[j] multiplies x[t - j]
#pragma unroll
  for (int j = 0; j < W; ++j)
#pragma unroll
    for (int i = 0; i < N; ++i) wr[j][i] = w[(int64_t)(c0 + i) * W + (W - 1 - j)];
  float hist[W > 1 ? W - 1 : 1][N];   // hist[j - 1] = x[t - j]
#pragma unroll
  for (int j = 1; j < W; ++j) {
    if (t0 - j >= 0) V::load(x + (t0 - j) * C + c0, hist[j - 1]);
    else
#pragma unroll
      for (int i = 0; i < N; ++i) hist[j - 1][i] = 0.f;
  }
  const int64_t t1 = min(t0 + kRows, T_);
  for (int64_t t = t0; t < t1; ++t) {
    float cur[N], acc[N];
    V::load(x + t * C + c0, cur);
    const int64_t p = pos != nullptr ? pos[t] : t;
#pragma unroll
    for (int i = 0; i < N; ++i) acc[i] = cur[i] * wr[0][i];
#pragma unroll
    for (int j = 1; j < W; ++j)
      if (p >= j)
#pragma unroll
        for (int i = 0; i < N; ++i) acc[i] += hist[j - 1][i] * wr[j][i];
#pragma unroll
    for (int i = 0; i < N; ++i) acc[i] = acc[i] / (1.f + __expf(-acc[i]));
    V::store(y + t * C + c0, acc);
#pragma unroll
    for (int j = W - 1; j > 1; --j)
#pragma unroll
      for (int i = 0; i < N; ++i) hist[j - 1][i] = hist[j - 2][i];
    if (W > 1)
#pragma unroll
      for (int i = 0; i < N; ++i) hist[0][i] = cur[i];
  }
}

// dx[t'] = sum_j w[W-1-j] * ds[t'+j] * [pos[t'+j] >= j];  dw[c, W-1-j] = sum_t ds[t] * x[t-j] * [pos[t] >= j].
template <typename T, int W>
__global__ void __launch_bounds__(kThreads)
conv_silu_bwd_kernel(const T* __restrict__ x, const float* __restrict__ w, const int64_t* __restrict__ pos,
                     const T* __restrict__ dy, T* __restrict__ dx, float* __restrict__ dw_part, int64_t T_, int C) {
  using V = ChanVec<T>;
  constexpr int N = V::N;
  const int cg = blockIdx.x * kThreads + threadIdx.x;
  if (cg * N >= C) return;
  const int c0 = cg * N;
  const int64_t t0 = (int64_t)blockIdx.y * kRows;
  float wr[W][N];
#pragma unroll
  for (int j = 0; j < W; ++j)
#pragma unroll
    for (int i = 0; i < N; ++i) wr[j][i] = w[(int64_t)(c0 + i) * W + (W - 1 - j)];
  float xh[W > 1 ? W - 1 : 1][N];   // xh[j - 1] = x[t - j]
#pragma unroll
  for (int j = 1; j < W; ++j) {
    if (t0 - j >= 0) V::load(x + (t0 - j) * C + c0, xh[j - 1]);
    else
#pragma unroll
      for (int i = 0; i < N; ++i) xh[j - 1][i] = 0.f;
  }
  float dsh[W][N];        // dsh[k] = ds[t - k] after row t has been processed
  int64_t ph[W];          // positions of the same rows
#pragma unroll
  for (int k = 0; k < W; ++k) {
    ph[k] = 0;
#pragma unroll
    for (int i = 0; i < N; ++i) dsh[k][i] = 0.f;
  }
  float dwa[W][N];
#pragma unroll
  for (int j = 0; j < W; ++j)
#pragma unroll
    for (int i = 0; i < N; ++i) dwa[j][i] = 0.f;
  const int64_t own_end = min(t0 + kRows, T_);
  // rows t0 .. own_end + W - 2: the last W - 1 only feed dx of the block's last rows
  for (int64_t t = t0; t < own_end + W - 1; ++t) {
    float ds[N];
    int64_t p = 0;
    float cur[N];
    if (t < T_) {
      float pre[N], g[N];
      V::load(x + t * C + c0, cur);
      V::load(dy + t * C + c0, g);
      p = pos != nullptr ? pos[t] : t;
#pragma unroll
      for (int i = 0; i < N; ++i) pre[i] = cur[i] * wr[0][i];
#pragma unroll
      for (int j = 1; j < W; ++j)
        if (p >= j)
#pragma unroll
          for (int i = 0; i < N; ++i) pre[i] += xh[j - 1][i] * wr[j][i];
#pragma unroll
      for (int i = 0; i < N; ++i) {
        const float s = 1.f / (1.f + __expf(-pre[i]));
        ds[i] = g[i] * (s + pre[i] * s * (1.f - s));
      }
      if (t < own_end) {   // this block owns row t's contribution to dw
#pragma unroll
        for (int i = 0; i < N; ++i) dwa[0][i] += ds[i] * cur[i];
#pragma unroll
        for (int j = 1; j < W; ++j)
          if (p >= j)
#pragma unroll
            for (int i = 0; i < N; ++i) dwa[j][i] += ds[i] * xh[j - 1][i];
      }
    } else {
#pragma unroll
      for (int i = 0; i < N; ++i) { ds[i] = 0.f; cur[i] = 0.f; }
    }
    // slide the ds window: dsh[0] = ds[t], dsh[k] = ds[t - k]
#pragma unroll
    for (int k = W - 1; k > 0; --k) {
      ph[k] = ph[k - 1];
#pragma unroll
      for (int i = 0; i < N; ++i) dsh[k][i] = dsh[k - 1][i];
    }
    ph[0] = p;
#pragma unroll
    for (int i = 0; i < N; ++i) dsh[0][i] = ds[i];
    // row t' = t - (W - 1) now has all of ds[t' .. t' + W - 1]:  ds[t' + j] = dsh[W - 1 - j]
    const int64_t tp = t - (W - 1);
    if (tp >= t0 && tp < own_end) {
      float acc[N];
#pragma unroll
      for (int i = 0; i < N; ++i) acc[i] = 0.f;
#pragma unroll
      for (int j = 0; j < W; ++j) {
        const bool live = (tp + j < T_) && (ph[W - 1 - j] >= j);
        if (live)
#pragma unroll
          for (int i = 0; i < N; ++i) acc[i] += wr[j][i] * dsh[W - 1 - j][i];
      }
      V::store(dx + tp * C + c0, acc);
    }
    // slide the x window
#pragma unroll
    for (int j = W - 1; j > 1; --j)
#pragma unroll
      for (int i = 0; i < N; ++i) xh[j - 1][i] = xh[j - 2][i];
    if (W > 1)
#pragma unroll
      for (int i = 0; i < N; ++i) xh[0][i] = cur[i];
  }
  float* out = dw_part + ((int64_t)blockIdx.y * C + c0) * W;
#pragma unroll
  for (int i = 0; i < N; ++i)
#pragma unroll
    for (int j = 0; j < W; ++j) out[i * W + (W - 1 - j)] = dwa[j][i];
}

void check(const at::Tensor& x, const at::Tensor& w, const c10::optional<at::Tensor>& pos) {
  TORCH_CHECK(x.is_cuda() && x.dim() == 2 && x.is_contiguous() &&
                  (x.scalar_type() == at::kBFloat16 || x.scalar_type() == at::kFloat),
              "conv_silu: x must be a contiguous [T, C] bf16 / fp32 CUDA tensor");
  TORCH_CHECK(w.is_cuda() && w.dim() == 2 && w.is_contiguous() && w.scalar_type() == at::kFloat && w.size(0) == x.size(1) &&
                  w.size(1) >= 1 && w.size(1) <= kMaxW,
              "conv_silu: w must be a contiguous fp32 [C, W] tensor with W <= 4");
  const int n = x.scalar_type() == at::kBFloat16 ? 8 : 4;
  TORCH_CHECK(x.size(1) % n == 0, "conv_silu: the channel count must be a multiple of ", n);
  if (pos.has_value() && pos->defined())
    TORCH_CHECK(pos->is_cuda() && pos->scalar_type() == at::kLong && pos->is_contiguous() && pos->numel() == x.size(0),
                "conv_silu: positions must be an int64 [T] CUDA tensor");
}

#define TB_CONV_DISPATCH(W_, ...)                          \
  switch (W_) {                                            \
    case 1: { constexpr int kW = 1; __VA_ARGS__; break; }  \
    case 2: { constexpr int kW = 2; __VA_ARGS__; break; }  \
    case 3: { constexpr int kW = 3; __VA_ARGS__; break; }  \
    default: { constexpr int kW = 4; __VA_ARGS__; break; } \
  }

}  // namespace

at::Tensor conv_silu_fwd(const at::Tensor& x, const at::Tensor& w, const c10::optional<at::Tensor>& pos) {
  check(x, w, pos);
  c10::cuda::CUDAGuard guard(x.device());
  auto y = at::empty_like(x);
  const int64_t T_ = x.size(0);
  const int C = (int)x.size(1);
  if (T_ == 0 || C == 0) return y;
  const int n = x.scalar_type() == at::kBFloat16 ? 8 : 4;
  const dim3 grid((unsigned)((C / n + kThreads - 1) / kThreads), (unsigned)((T_ + kRows - 1) / kRows));
  const int64_t* pp = (pos.has_value() && pos->defined()) ? pos->data_ptr<int64_t>() : nullptr;
  auto stream = at::cuda::getCurrentCUDAStream();
  const int W = (int)w.size(1);
  if (x.scalar_type() == at::kBFloat16) {
    using T = __nv_bfloat16;
    TB_CONV_DISPATCH(W, (conv_silu_fwd_kernel<T, kW><<<grid, kThreads, 0, stream>>>(
        reinterpret_cast<const T*>(x.data_ptr()), w.data_ptr<float>(), pp, reinterpret_cast<T*>(y.data_ptr()), T_, C)));
  } else {
    TB_CONV_DISPATCH(W, (conv_silu_fwd_kernel<float, kW><<<grid, kThreads, 0, stream>>>(
        x.data_ptr<float>(), w.data_ptr<float>(), pp, y.data_ptr<float>(), T_, C)));
  }
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  return y;
}

// Returns (dx [T, C], dw [C, W] fp32).
std::tuple<at::Tensor, at::Tensor> conv_silu_bwd(const at::Tensor& x, const at::Tensor& w,
                                                 const c10::optional<at::Tensor>& pos, const at::Tensor& dy) {
  check(x, w, pos);
  TORCH_CHECK(dy.is_cuda() && dy.is_contiguous() && dy.sizes() == x.sizes() && dy.scalar_type() == x.scalar_type());
  c10::cuda::CUDAGuard guard(x.device());
  auto dx = at::empty_like(x);
  const int64_t T_ = x.size(0);
  const int C = (int)x.size(1);
  const int W = (int)w.size(1);
  if (T_ == 0 || C == 0) return {dx, at::zeros({C, W}, w.options())};
  const int n = x.scalar_type() == at::kBFloat16 ? 8 : 4;
  const int64_t nblk = (T_ + kRows - 1) / kRows;
  auto part = at::empty({nblk, C, W}, w.options());
  const dim3 grid((unsigned)((C / n + kThreads - 1) / kThreads), (unsigned)nblk);
  const int64_t* pp = (pos.has_value() && pos->defined()) ? pos->data_ptr<int64_t>() : nullptr;
  auto stream = at::cuda::getCurrentCUDAStream();
  if (x.scalar_type() == at::kBFloat16) {
    using T = __nv_bfloat16;
    TB_CONV_DISPATCH(W, (conv_silu_bwd_kernel<T, kW><<<grid, kThreads, 0, stream>>>(
        reinterpret_cast<const T*>(x.data_ptr()), w.data_ptr<float>(), pp, reinterpret_cast<const T*>(dy.data_ptr()),
        reinterpret_cast<T*>(dx.data_ptr()), part.data_ptr<float>(), T_, C)));
  } else {
    TB_CONV_DISPATCH(W, (conv_silu_bwd_kernel<float, kW><<<grid, kThreads, 0, stream>>>(
        x.data_ptr<float>(), w.data_ptr<float>(), pp, dy.data_ptr<float>(), dx.data_ptr<float>(), part.data_ptr<float>(),
        T_, C)));
  }
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  return {dx, part.sum(0)};
}

}  // namespace tb200
