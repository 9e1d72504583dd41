// Bandwidth-bound operators: RMSNorm fwd/bwd, RoPE (in place), SwiGLU fwd/bwd.
//
// All kernels move 16 bytes per thread per access, do their math in fp32 and are
// sized so that a wave fills the 148 SMs; none of them allocates or waits on
// another kernel.  Row lengths must be multiples of the 16-byte vector width
// (checked on the host), which also gives the required alignment.
#include <ATen/ATen.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/library.h>

#include "common.cuh"

namespace tb200 {

__device__ int g_status_word = 0;

template <typename T>
struct Vec16;
template <>
struct Vec16<__nv_bfloat16> {
  static constexpr int N = 8;
  bf16x8 raw;
  __device__ __forceinline__ void load(const __nv_bfloat16* p) { raw = *reinterpret_cast<const bf16x8*>(p); }
  __device__ __forceinline__ void store(__nv_bfloat16* p) const { *reinterpret_cast<bf16x8*>(p) = raw; }
  __device__ __forceinline__ void get(float (&f)[8]) const { unpack8(raw, f); }
  __device__ __forceinline__ void set(const float (&f)[8]) { raw = pack8(f); }
};
template <>
struct Vec16<float> {
  static constexpr int N = 4;
  float4 raw;
  __device__ __forceinline__ void load(const float* p) { raw = *reinterpret_cast<const float4*>(p); }
  __device__ __forceinline__ void store(float* p) const { *reinterpret_cast<float4*>(p) = raw; }
  __device__ __forceinline__ void get(float (&f)[4]) const { f[0] = raw.x; f[1] = raw.y; f[2] = raw.z; f[3] = raw.w; }
  __device__ __forceinline__ void set(const float (&f)[4]) { raw = make_float4(f[0], f[1], f[2], f[3]); }
};

// ----------------------------------------------------------------------------
// RMSNorm.  A row is handled by a *group* of threads: one warp (kWarpRow, several
// rows per CTA, for short rows such as per-head QK-norm) or the whole CTA.  Each
// thread keeps VPT 16-byte vectors of the row in registers between the reduction
// and the scaling pass, so x is read from HBM exactly once.
// ----------------------------------------------------------------------------
template <bool kWarpRow>
__device__ __forceinline__ float group_sum(float v, float* red) {
  if (kWarpRow) return warp_sum(v);
  return block_sum(v, red);
}

template <typename T, bool kHasWeight, int VPT, bool kWarpRow>
__global__ void __launch_bounds__(512) rmsnorm_fwd_kernel(const T* __restrict__ x, const T* __restrict__ w,
                                                           T* __restrict__ y, float* __restrict__ rstd_out,
                                                           int64_t rows, int D, float eps) {
  using V = Vec16<T>;
  constexpr int N = V::N;
  __shared__ float red[32];
  const int gsize = kWarpRow ? 32 : blockDim.x;
  const int gid = kWarpRow ? (threadIdx.x >> 5) : 0;
  const int gpb = kWarpRow ? (blockDim.x >> 5) : 1;
  const int t = kWarpRow ? (threadIdx.x & 31) : threadIdx.x;
  const int nvec = D / N;
  for (int64_t row = (int64_t)blockIdx.x * gpb + gid; row < rows; row += (int64_t)gridDim.x * gpb) {
    const T* xr = x + row * D;
    T* yr = y + row * D;
    V cache[VPT];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int v = t + i * gsize;
      if (v < nvec) {
        cache[i].load(xr + v * N);
        float f[N];
        cache[i].get(f);
#pragma unroll
        for (int j = 0; j < N; ++j) ss += f[j] * f[j];
      }
    }
    ss = group_sum<kWarpRow>(ss, red);
    const float rstd = rsqrtf(ss / (float)D + eps);
    if (t == 0) rstd_out[row] = rstd;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int v = t + i * gsize;
      if (v < nvec) {
        float f[N];
        cache[i].get(f);
        if (kHasWeight) {
          V wv;
          wv.load(w + v * N);
          float g[N];
          wv.get(g);
#pragma unroll
          for (int j = 0; j < N; ++j) f[j] = f[j] * rstd * g[j];
        } else {
#pragma unroll
          for (int j = 0; j < N; ++j) f[j] *= rstd;
        }
        V o;
        o.set(f);
        o.store(yr + v * N);
      }
    }
  }
}

// Backward.  A persistent grid walks the rows; every group keeps the weight-gradient
// partial sums of its columns in registers and writes them once to
// `dw_partial[num_groups, D]`; a second kernel reduces the partials.
//   xhat = x * rstd ; g = dy * w ; c = mean(g * xhat) ; dx = (g - xhat * c) * rstd
template <typename T, bool kHasWeight, int VPT, bool kWarpRow>
__global__ void __launch_bounds__(512) rmsnorm_bwd_kernel(const T* __restrict__ dy, const T* __restrict__ x,
                                                           const T* __restrict__ w, const float* __restrict__ rstd_in,
                                                           T* __restrict__ dx, float* __restrict__ dw_partial,
                                                           int64_t rows, int D) {
  using V = Vec16<T>;
  constexpr int N = V::N;
  __shared__ float red[32];
  const int gsize = kWarpRow ? 32 : blockDim.x;
  const int gid = kWarpRow ? (threadIdx.x >> 5) : 0;
  const int gpb = kWarpRow ? (blockDim.x >> 5) : 1;
  const int t = kWarpRow ? (threadIdx.x & 31) : threadIdx.x;
  const int nvec = D / N;
  float dwacc[VPT][N];
#pragma unroll
  for (int i = 0; i < VPT; ++i)
#pragma unroll
    for (int j = 0; j < N; ++j) dwacc[i][j] = 0.f;
  // Every group runs the same number of iterations so that block-wide reductions stay aligned.
  const int64_t stride = (int64_t)gridDim.x * gpb;
  const int64_t iters = (rows + stride - 1) / stride;
  for (int64_t it = 0; it < iters; ++it) {
    const int64_t row = it * stride + (int64_t)blockIdx.x * gpb + gid;
    const bool live = row < rows;
    float xh[VPT][N], g[VPT][N];
    float dot = 0.f;
    float rstd = 0.f;
    if (live) {
      rstd = rstd_in[row];
      const T* xr = x + row * D;
      const T* dyr = dy + row * D;
#pragma unroll
      for (int i = 0; i < VPT; ++i) {
        const int v = t + i * gsize;
        if (v < nvec) {
          V xv, dv;
          xv.load(xr + v * N);
          dv.load(dyr + v * N);
          float xf[N], df[N], wf[N];
          xv.get(xf);
          dv.get(df);
          if (kHasWeight) {
            V wv;
            wv.load(w + v * N);
            wv.get(wf);
          }
#pragma unroll
          for (int j = 0; j < N; ++j) {
            xh[i][j] = xf[j] * rstd;
            if (kHasWeight) {
              dwacc[i][j] += df[j] * xh[i][j];
              g[i][j] = df[j] * wf[j];
            } else {
              g[i][j] = df[j];
            }
            dot += g[i][j] * xh[i][j];
          }
        }
      }
    }
    dot = group_sum<kWarpRow>(dot, red);
    if (live) {
      const float c = dot / (float)D;
      T* dxr = dx + row * D;
#pragma unroll
      for (int i = 0; i < VPT; ++i) {
        const int v = t + i * gsize;
        if (v < nvec) {
          float o[N];
#pragma unroll
          for (int j = 0; j < N; ++j) o[j] = (g[i][j] - xh[i][j] * c) * rstd;
          V ov;
          ov.set(o);
          ov.store(dxr + v * N);
        }
      }
    }
  }
  if (kHasWeight) {
    float* out = dw_partial + ((int64_t)blockIdx.x * gpb + gid) * D;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int v = t + i * gsize;
      if (v < nvec) {
#pragma unroll
        for (int j = 0; j < N; ++j) out[v * N + j] = dwacc[i][j];
      }
    }
  }
}

// Column sums of partial[nparts, D]: a 32x8 thread tile per 32 columns, rows split over the
// 8 thread rows, then a shared-memory reduction.  D/32 CTAs.
__global__ void __launch_bounds__(256) colsum_kernel(const float* __restrict__ partial, float* __restrict__ out,
                                                     int nparts, int D) {
  __shared__ float tile[8][33];
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  const int col = blockIdx.x * 32 + tx;
  float s = 0.f;
  if (col < D) {
    for (int p = ty; p < nparts; p += 8) s += partial[(int64_t)p * D + col];
  }
  tile[ty][tx] = s;
  __syncthreads();
  if (ty == 0 && col < D) {
    float t = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) t += tile[i][tx];
    out[col] = t;
  }
}

// ----------------------------------------------------------------------------
// RoPE in place on x[T, H, D] (row stride in elements, heads contiguous).
// `table[P, rot]` holds cos | sin (fp32).  interleaved: pairs (2i, 2i+1); otherwise
// pairs (i, i + rot/2).  `inverse` applies the transposed rotation (backward).
// A position outside the table is clamped and reported in the status word.
// ----------------------------------------------------------------------------
template <typename T, bool kInterleaved>
__global__ void __launch_bounds__(256) rope_kernel(T* __restrict__ x, const float* __restrict__ table,
                                                   const int64_t* __restrict__ positions, int64_t T_rows, int H, int D,
                                                   int64_t row_stride, int rot, int P, float sign) {
  using V = Vec16<T>;
  constexpr int N = V::N;
  const int half = rot / 2;
  // work item = (row, head, vector of the first half of pairs)
  const int items_per_head = kInterleaved ? (rot / N) : (half / N);
  const int64_t total = T_rows * H * items_per_head;
  for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (int64_t)gridDim.x * blockDim.x) {
    const int it = (int)(idx % items_per_head);
    const int64_t rh = idx / items_per_head;
    const int h = (int)(rh % H);
    const int64_t row = rh / H;
    int64_t pos = positions[row];
    if (pos < 0 || pos >= P) {
      atomicOr(&g_status_word, kStatusRopePositionOutOfRange);
      pos = pos < 0 ? 0 : P - 1;
    }
    const float* cs = table + pos * rot;
    T* base = x + row * row_stride + (int64_t)h * D;
    if (kInterleaved) {
      V v;
      v.load(base + it * N);
      float f[N];
      v.get(f);
      const int p0 = it * (N / 2);
#pragma unroll
      for (int j = 0; j < N / 2; ++j) {
        const float c = cs[p0 + j], s = sign * cs[half + p0 + j];
        const float a = f[2 * j], b = f[2 * j + 1];
        f[2 * j] = a * c - b * s;
        f[2 * j + 1] = a * s + b * c;
      }
      v.set(f);
      v.store(base + it * N);
    } else {
      V lo, hi;
      lo.load(base + it * N);
      hi.load(base + half + it * N);
      float a[N], b[N];
      lo.get(a);
      hi.get(b);
#pragma unroll
      for (int j = 0; j < N; ++j) {
        const float c = cs[it * N + j], s = sign * cs[half + it * N + j];
        const float u = a[j], w = b[j];
        a[j] = u * c - w * s;
        b[j] = w * c + u * s;
      }
      lo.set(a);
      hi.set(b);
      lo.store(base + it * N);
      hi.store(base + half + it * N);
    }
  }
}

// ----------------------------------------------------------------------------
// SwiGLU on gate_up[T, 2F] = [gate | up].
// ----------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256) swiglu_fwd_kernel(const T* __restrict__ gu, T* __restrict__ out, int64_t rows,
                                                         int F) {
  using V = Vec16<T>;
  constexpr int N = V::N;
  const int vpr = F / N;
  const int64_t total = rows * vpr;
  for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (int64_t)gridDim.x * blockDim.x) {
    const int64_t row = idx / vpr;
    const int v = (int)(idx % vpr);
    V g, u;
    g.load(gu + row * 2 * F + v * N);
    u.load(gu + row * 2 * F + F + v * N);
    float gf[N], uf[N];
    g.get(gf);
    u.get(uf);
#pragma unroll
    for (int j = 0; j < N; ++j) {
      const float s = 1.f / (1.f + __expf(-gf[j]));
      gf[j] = gf[j] * s * uf[j];
    }
    V o;
    o.set(gf);
    o.store(out + row * F + v * N);
  }
}

template <typename T>
__global__ void __launch_bounds__(256) swiglu_bwd_kernel(const T* __restrict__ gu, const T* __restrict__ dout,
                                                         T* __restrict__ dgu, int64_t rows, int F) {
  using V = Vec16<T>;
  constexpr int N = V::N;
  const int vpr = F / N;
  const int64_t total = rows * vpr;
  for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (int64_t)gridDim.x * blockDim.x) {
    const int64_t row = idx / vpr;
    const int v = (int)(idx % vpr);
    V g, u, d;
    g.load(gu + row * 2 * F + v * N);
    u.load(gu + row * 2 * F + F + v * N);
    d.load(dout + row * F + v * N);
    float gf[N], uf[N], df[N];
    g.get(gf);
    u.get(uf);
    d.get(df);
#pragma unroll
    for (int j = 0; j < N; ++j) {
      const float s = 1.f / (1.f + __expf(-gf[j]));
      const float silu = gf[j] * s;
      const float dg = df[j] * uf[j] * (s + silu * (1.f - s));
      const float du = df[j] * silu;
      gf[j] = dg;
      uf[j] = du;
    }
    g.set(gf);
    u.set(uf);
    g.store(dgu + row * 2 * F + v * N);
    u.store(dgu + row * 2 * F + F + v * N);
  }
}

// ============================================================================
// host side
// ============================================================================
static inline int grid_for(int64_t work_items, int threads, int ctas_per_sm = 8) {
  const int64_t want = (work_items + threads - 1) / threads;
  const int64_t cap = (int64_t)num_sms() * ctas_per_sm;
  return (int)std::max<int64_t>(1, std::min<int64_t>(want, cap));
}

#define TB_DISPATCH_FLOAT(dtype, ...)                                   \
  if ((dtype) == at::kBFloat16) {                                       \
    using scalar_t = __nv_bfloat16;                                     \
    __VA_ARGS__();                                                      \
  } else if ((dtype) == at::kFloat) {                                   \
    using scalar_t = float;                                             \
    __VA_ARGS__();                                                      \
  } else {                                                              \
    TORCH_CHECK(false, "tb200: unsupported dtype ", (dtype));           \
  }

struct RowPlan {
  bool warp_row;
  int vpt;
  int threads;
  int groups_per_block;
};

// Short rows: one warp per row, 8 rows per CTA.  Long rows: the CTA per row, with 1, 2 or 4
// vectors per thread.
static RowPlan plan_row(int nvec) {
  RowPlan p;
  if (nvec <= 128) {
    p.warp_row = true;
    p.vpt = nvec <= 32 ? 1 : (nvec <= 64 ? 2 : 4);
    p.threads = 256;
    p.groups_per_block = 8;
    return p;
  }
  p.warp_row = false;
  p.vpt = nvec <= 256 ? 1 : (nvec <= 512 ? 2 : 4);
  int t = (nvec + p.vpt - 1) / p.vpt;
  t = (t + 31) / 32 * 32;
  p.threads = t;
  p.groups_per_block = 1;
  return p;
}

#define TB_DISPATCH_PLAN(plan, ...)                                              \
  if ((plan).warp_row) {                                                         \
    constexpr bool kWarpRow = true;                                              \
    if ((plan).vpt == 1) { constexpr int VPT = 1; __VA_ARGS__(); }               \
    else if ((plan).vpt == 2) { constexpr int VPT = 2; __VA_ARGS__(); }          \
    else { constexpr int VPT = 4; __VA_ARGS__(); }                               \
  } else {                                                                       \
    constexpr bool kWarpRow = false;                                             \
    if ((plan).vpt == 1) { constexpr int VPT = 1; __VA_ARGS__(); }               \
    else if ((plan).vpt == 2) { constexpr int VPT = 2; __VA_ARGS__(); }          \
    else { constexpr int VPT = 4; __VA_ARGS__(); }                               \
  }

std::tuple<at::Tensor, at::Tensor> rmsnorm_fwd(const at::Tensor& x, const c10::optional<at::Tensor>& w, double eps) {
  TORCH_CHECK(x.is_cuda() && x.dim() == 2 && x.is_contiguous(), "rmsnorm_fwd: x must be a contiguous CUDA matrix");
  const int64_t rows = x.size(0);
  const int D = (int)x.size(1);
  const int vecw = x.scalar_type() == at::kBFloat16 ? 8 : 4;
  TORCH_CHECK(D % vecw == 0, "rmsnorm_fwd: row length must be a multiple of ", vecw);
  TORCH_CHECK(D / vecw <= 2048, "rmsnorm_fwd: row length ", D, " exceeds the register-resident limit");
  if (w.has_value()) TORCH_CHECK(w->is_contiguous() && w->numel() == D && w->scalar_type() == x.scalar_type());
  c10::cuda::CUDAGuard guard(x.device());
  auto y = at::empty_like(x);
  auto rstd = at::empty({rows}, x.options().dtype(at::kFloat));
  if (rows == 0) return {y, rstd};
  auto stream = at::cuda::getCurrentCUDAStream();
  const RowPlan plan = plan_row(D / vecw);
  const int64_t want = (rows + plan.groups_per_block - 1) / plan.groups_per_block;
  const int grid = (int)std::min<int64_t>(want, (int64_t)num_sms() * 64);
  TB_DISPATCH_FLOAT(x.scalar_type(), [&] {
    auto xp = reinterpret_cast<const scalar_t*>(x.data_ptr());
    auto yp = reinterpret_cast<scalar_t*>(y.data_ptr());
    auto wp = w.has_value() ? reinterpret_cast<const scalar_t*>(w->data_ptr()) : nullptr;
    TB_DISPATCH_PLAN(plan, [&] {
      if (w.has_value()) {
        rmsnorm_fwd_kernel<scalar_t, true, VPT, kWarpRow><<<grid, plan.threads, 0, stream>>>(
            xp, wp, yp, rstd.data_ptr<float>(), rows, D, (float)eps);
      } else {
        rmsnorm_fwd_kernel<scalar_t, false, VPT, kWarpRow><<<grid, plan.threads, 0, stream>>>(
            xp, wp, yp, rstd.data_ptr<float>(), rows, D, (float)eps);
      }
    });
  });
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  return {y, rstd};
}

std::tuple<at::Tensor, at::Tensor> rmsnorm_bwd(const at::Tensor& dy, const at::Tensor& x,
                                               const c10::optional<at::Tensor>& w, const at::Tensor& rstd) {
  TORCH_CHECK(x.is_cuda() && x.dim() == 2 && x.is_contiguous() && dy.is_contiguous() && dy.sizes() == x.sizes());
  TORCH_CHECK(dy.scalar_type() == x.scalar_type() && rstd.scalar_type() == at::kFloat);
  const int64_t rows = x.size(0);
  const int D = (int)x.size(1);
  const int vecw = x.scalar_type() == at::kBFloat16 ? 8 : 4;
  TORCH_CHECK(D % vecw == 0);
  TORCH_CHECK(D / vecw <= 2048, "rmsnorm_bwd: row length ", D, " exceeds the register-resident limit");
  c10::cuda::CUDAGuard guard(x.device());
  auto dx = at::empty_like(x);
  auto dw = at::zeros({w.has_value() ? D : 0}, x.options().dtype(at::kFloat));
  if (rows == 0) return {dx, dw};
  auto stream = at::cuda::getCurrentCUDAStream();
  const RowPlan plan = plan_row(D / vecw);
  const int64_t want = (rows + plan.groups_per_block - 1) / plan.groups_per_block;
  const int per_sm = std::max(1, 2048 / plan.threads);
  const int grid = (int)std::min<int64_t>(want, (int64_t)num_sms() * per_sm);
  const int nparts = grid * plan.groups_per_block;
  at::Tensor partial;
  if (w.has_value()) partial = at::empty({nparts, D}, x.options().dtype(at::kFloat));
  TB_DISPATCH_FLOAT(x.scalar_type(), [&] {
    auto dyp = reinterpret_cast<const scalar_t*>(dy.data_ptr());
    auto xp = reinterpret_cast<const scalar_t*>(x.data_ptr());
    auto dxp = reinterpret_cast<scalar_t*>(dx.data_ptr());
    auto wp = w.has_value() ? reinterpret_cast<const scalar_t*>(w->data_ptr()) : nullptr;
    auto pp = w.has_value() ? partial.data_ptr<float>() : nullptr;
    TB_DISPATCH_PLAN(plan, [&] {
      if (w.has_value()) {
        rmsnorm_bwd_kernel<scalar_t, true, VPT, kWarpRow><<<grid, plan.threads, 0, stream>>>(
            dyp, xp, wp, rstd.data_ptr<float>(), dxp, pp, rows, D);
      } else {
        rmsnorm_bwd_kernel<scalar_t, false, VPT, kWarpRow><<<grid, plan.threads, 0, stream>>>(
            dyp, xp, wp, rstd.data_ptr<float>(), dxp, pp, rows, D);
      }
    });
  });
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  if (w.has_value()) {
    colsum_kernel<<<(D + 31) / 32, 256, 0, stream>>>(partial.data_ptr<float>(), dw.data_ptr<float>(), nparts, D);
    C10_CUDA_KERNEL_LAUNCH_CHECK();
  }
  return {dx, dw};
}

void rope_(at::Tensor x, const at::Tensor& table, const at::Tensor& positions, bool interleaved, bool inverse) {
  TORCH_CHECK(x.is_cuda() && x.dim() == 3 && x.stride(2) == 1, "rope_: x must be [T, H, D] with contiguous D");
  TORCH_CHECK(x.stride(1) == x.size(2), "rope_: heads must be adjacent");
  TORCH_CHECK(table.scalar_type() == at::kFloat && table.is_contiguous() && table.dim() == 2);
  TORCH_CHECK(positions.scalar_type() == at::kLong && positions.is_contiguous() && positions.numel() == x.size(0));
  const int D = (int)x.size(2), H = (int)x.size(1);
  const int rot = (int)table.size(1);
  const int vecw = x.scalar_type() == at::kBFloat16 ? 8 : 4;
  TORCH_CHECK(rot <= D && rot % 2 == 0);
  TORCH_CHECK(interleaved ? (rot % vecw == 0) : ((rot / 2) % vecw == 0), "rope_: rotary width not vectorisable");
  TORCH_CHECK(x.stride(0) % vecw == 0 && D % vecw == 0 && (x.storage_offset() % vecw) == 0,
              "rope_: rows must be 16-byte aligned");
  if (x.numel() == 0) return;
  c10::cuda::CUDAGuard guard(x.device());
  auto stream = at::cuda::getCurrentCUDAStream();
  const int items_per_head = interleaved ? rot / vecw : (rot / 2) / vecw;
  const int64_t total = x.size(0) * H * items_per_head;
  const int grid = grid_for(total, 256);
  const float sign = inverse ? -1.f : 1.f;
  TB_DISPATCH_FLOAT(x.scalar_type(), [&] {
    auto xp = reinterpret_cast<scalar_t*>(x.data_ptr());
    if (interleaved) {
      rope_kernel<scalar_t, true><<<grid, 256, 0, stream>>>(xp, table.data_ptr<float>(), positions.data_ptr<int64_t>(),
                                                            x.size(0), H, D, x.stride(0), rot, (int)table.size(0), sign);
    } else {
      rope_kernel<scalar_t, false><<<grid, 256, 0, stream>>>(xp, table.data_ptr<float>(),
                                                             positions.data_ptr<int64_t>(), x.size(0), H, D,
                                                             x.stride(0), rot, (int)table.size(0), sign);
    }
  });
  C10_CUDA_KERNEL_LAUNCH_CHECK();
}

at::Tensor swiglu_fwd(const at::Tensor& gu) {
  TORCH_CHECK(gu.is_cuda() && gu.dim() == 2 && gu.is_contiguous() && gu.size(1) % 2 == 0);
  const int F = (int)(gu.size(1) / 2);
  const int vecw = gu.scalar_type() == at::kBFloat16 ? 8 : 4;
  TORCH_CHECK(F % vecw == 0, "swiglu: hidden size must be a multiple of ", vecw);
  c10::cuda::CUDAGuard guard(gu.device());
  auto out = at::empty({gu.size(0), F}, gu.options());
  if (out.numel() == 0) return out;
  auto stream = at::cuda::getCurrentCUDAStream();
  const int grid = grid_for(gu.size(0) * (F / vecw), 256);
  TB_DISPATCH_FLOAT(gu.scalar_type(), [&] {
    swiglu_fwd_kernel<scalar_t><<<grid, 256, 0, stream>>>(reinterpret_cast<const scalar_t*>(gu.data_ptr()),
                                                          reinterpret_cast<scalar_t*>(out.data_ptr()), gu.size(0), F);
  });
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  return out;
}

at::Tensor swiglu_bwd(const at::Tensor& gu, const at::Tensor& dout) {
  TORCH_CHECK(gu.is_cuda() && gu.dim() == 2 && gu.is_contiguous() && dout.is_contiguous());
  const int F = (int)(gu.size(1) / 2);
  TORCH_CHECK(dout.size(0) == gu.size(0) && dout.size(1) == F && dout.scalar_type() == gu.scalar_type());
  const int vecw = gu.scalar_type() == at::kBFloat16 ? 8 : 4;
  TORCH_CHECK(F % vecw == 0);
  c10::cuda::CUDAGuard guard(gu.device());
  auto dgu = at::empty_like(gu);
  if (dgu.numel() == 0) return dgu;
  auto stream = at::cuda::getCurrentCUDAStream();
  const int grid = grid_for(gu.size(0) * (F / vecw), 256);
  TB_DISPATCH_FLOAT(gu.scalar_type(), [&] {
    swiglu_bwd_kernel<scalar_t><<<grid, 256, 0, stream>>>(
        reinterpret_cast<const scalar_t*>(gu.data_ptr()), reinterpret_cast<const scalar_t*>(dout.data_ptr()),
        reinterpret_cast<scalar_t*>(dgu.data_ptr()), gu.size(0), F);
  });
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  return dgu;
}

// Address of the status word on the current device, for kernels of other translation units.
int* status_word_ptr() {
  int* p = nullptr;
  C10_CUDA_CHECK(cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_status_word));
  return p;
}

int64_t status(bool clear) {
  int v = 0;
  cudaMemcpyFromSymbol(&v, g_status_word, sizeof(int));
  if (clear && v != 0) {
    int z = 0;
    cudaMemcpyToSymbol(g_status_word, &z, sizeof(int));
  }
  return v;
}

}  // namespace tb200
