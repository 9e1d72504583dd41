// Mixture-of-experts routing kernels (CUDA cores; the expert GEMMs are the grouped tcgen05 GEMM).
//
//  * router_fwd / router_bwd: fp32 gate logits [T, E] -> softmax or sigmoid scores, expert-bias
//    aware top-k selection, optional renormalisation and scaling of the selected scores, and the
//    per-expert token histogram.  One warp per token, the score row lives in registers.
//  * permute_rows: tokens [T, D] -> expert-major padded layout [R, D] (row `dest[t, k]` receives
//    token t; rows that no slot maps to stay zero).
//  * combine_rows: out[t] = sum_k w[t, k] * y[dest[t, k]] in fp32, no atomics (deterministic), and
//    its two gradients (scatter of w * dout, and dw = <dout[t], y[dest]>).
#include <ATen/ATen.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>

#include "common.cuh"

namespace tb200 {

constexpr int kMaxExpertsPerLane = 16;   // experts <= 512
constexpr int kMaxTopK = 16;

struct RouterArgs {
  int T, E, K;
  int sigmoid;
  int route_norm;
  float route_scale;
};

template <int kPerLane>
__device__ __forceinline__ void router_scores(const float* __restrict__ row, int E, int lane, bool sigmoid,
                                              float (&s)[kPerLane]) {
  float m = -INFINITY;
#pragma unroll
  for (int i = 0; i < kPerLane; ++i) {
    const int e = i * 32 + lane;
    s[i] = e < E ? row[e] : -INFINITY;
    m = fmaxf(m, s[i]);
  }
  if (sigmoid) {
#pragma unroll
    for (int i = 0; i < kPerLane; ++i) s[i] = (i * 32 + lane) < E ? 1.f / (1.f + __expf(-s[i])) : 0.f;
    return;
  }
  m = warp_max(m);
  float sum = 0.f;
#pragma unroll
  for (int i = 0; i < kPerLane; ++i) {
    s[i] = (i * 32 + lane) < E ? __expf(s[i] - m) : 0.f;
    sum += s[i];
  }
  sum = warp_sum(sum);
  const float inv = 1.f / sum;
#pragma unroll
  for (int i = 0; i < kPerLane; ++i) s[i] *= inv;
}

template <int kPerLane>
__global__ void router_fwd_kernel(const float* __restrict__ logits, const float* __restrict__ bias,
                                  float* __restrict__ top, int* __restrict__ sel, float* __restrict__ counts,
                                  RouterArgs a) {
  const int64_t w = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (w >= a.T) return;
  float s[kPerLane], c[kPerLane];
  router_scores<kPerLane>(logits + w * a.E, a.E, lane, a.sigmoid != 0, s);
#pragma unroll
  for (int i = 0; i < kPerLane; ++i) {
    const int e = i * 32 + lane;
    c[i] = e < a.E ? s[i] + (bias != nullptr ? bias[e] : 0.f) : -INFINITY;
  }
  float picked[kMaxTopK];
  int picked_e[kMaxTopK];
  float total = 0.f;
  for (int k = 0; k < a.K; ++k) {
    // lane-local best (lowest expert index wins ties), then across the warp
    float bv = -INFINITY, bs = 0.f;
    int be = 0x7fffffff;
#pragma unroll
    for (int i = 0; i < kPerLane; ++i) {
      const int e = i * 32 + lane;
      if (c[i] > bv) { bv = c[i]; be = e; bs = s[i]; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int oe = __shfl_xor_sync(0xffffffffu, be, o);
      const float os = __shfl_xor_sync(0xffffffffu, bs, o);
      if (ov > bv || (ov == bv && oe < be)) { bv = ov; be = oe; bs = os; }
    }
    picked[k] = bs;
    picked_e[k] = be;
    total += bs;
#pragma unroll
    for (int i = 0; i < kPerLane; ++i)
      if (i * 32 + lane == be) c[i] = -INFINITY;
  }
  if (lane == 0) {
    const float norm = a.route_norm ? 1.f / (total + 1e-20f) : 1.f;
    for (int k = 0; k < a.K; ++k) {
      top[w * a.K + k] = picked[k] * norm * a.route_scale;
      sel[w * a.K + k] = picked_e[k];
      atomicAdd(counts + picked_e[k], 1.0f);   // integer-valued: the sum does not depend on the order
    }
  }
}

// dlogits from dtop: through the scaling / renormalisation, the gather and the score function.
template <int kPerLane>
__global__ void router_bwd_kernel(const float* __restrict__ logits, const int* __restrict__ sel,
                                  const float* __restrict__ dtop, float* __restrict__ dlogits, RouterArgs a) {
  const int64_t w = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (w >= a.T) return;
  float s[kPerLane], ds[kPerLane];
  router_scores<kPerLane>(logits + w * a.E, a.E, lane, a.sigmoid != 0, s);
#pragma unroll
  for (int i = 0; i < kPerLane; ++i) ds[i] = 0.f;
  // every lane walks the K selected experts (K is small) and keeps what lands on its own experts
  float raw_sum = 0.f, dot = 0.f;
  for (int k = 0; k < a.K; ++k) {
    const int e = sel[w * a.K + k];
    float mine = 0.f;
#pragma unroll
    for (int i = 0; i < kPerLane; ++i)
      if (i == (e >> 5)) mine = s[i];
    const float raw = __shfl_sync(0xffffffffu, mine, e & 31);
    raw_sum += raw;
    dot += dtop[w * a.K + k] * raw;
  }
  const float S = raw_sum + 1e-20f;
  for (int k = 0; k < a.K; ++k) {
    const int e = sel[w * a.K + k];
    const float g = dtop[w * a.K + k];
    const float draw = a.route_norm ? a.route_scale * (g / S - dot / (S * S)) : a.route_scale * g;
    if ((e & 31) == lane) {
#pragma unroll
      for (int i = 0; i < kPerLane; ++i)
        if (i == (e >> 5)) ds[i] += draw;
    }
  }
  if (a.sigmoid) {
#pragma unroll
    for (int i = 0; i < kPerLane; ++i) {
      const int e = i * 32 + lane;
      if (e < a.E) dlogits[w * a.E + e] = ds[i] * s[i] * (1.f - s[i]);
    }
  } else {
    float inner = 0.f;
#pragma unroll
    for (int i = 0; i < kPerLane; ++i) inner += ds[i] * s[i];
    inner = warp_sum(inner);
#pragma unroll
    for (int i = 0; i < kPerLane; ++i) {
      const int e = i * 32 + lane;
      if (e < a.E) dlogits[w * a.E + e] = s[i] * (ds[i] - inner);
    }
  }
}

template <typename F>
static void dispatch_per_lane(int E, F&& f) {
  if (E <= 64) f(std::integral_constant<int, 2>());
  else if (E <= 128) f(std::integral_constant<int, 4>());
  else if (E <= 256) f(std::integral_constant<int, 8>());
  else f(std::integral_constant<int, kMaxExpertsPerLane>());
}

std::tuple<at::Tensor, at::Tensor, at::Tensor> moe_router_fwd(const at::Tensor& logits, const c10::optional<at::Tensor>& bias,
                                                              int64_t top_k, bool sigmoid, bool route_norm,
                                                              double route_scale) {
  TORCH_CHECK(logits.is_cuda() && logits.scalar_type() == at::kFloat && logits.dim() == 2 && logits.is_contiguous());
  const int64_t T = logits.size(0), E = logits.size(1);
  TORCH_CHECK(E <= 32 * kMaxExpertsPerLane && top_k >= 1 && top_k <= kMaxTopK && top_k <= E, "moe_router: unsupported E or top_k");
  c10::cuda::CUDAGuard guard(logits.device());
  auto top = at::empty({T, top_k}, logits.options());
  auto sel = at::empty({T, top_k}, logits.options().dtype(at::kInt));
  auto counts = at::zeros({E}, logits.options());
  if (T == 0) return {top, sel, counts};
  const float* bp = nullptr;
  if (bias.has_value() && bias->defined()) {
    TORCH_CHECK(bias->is_cuda() && bias->scalar_type() == at::kFloat && bias->numel() == E && bias->is_contiguous());
    bp = bias->data_ptr<float>();
  }
  RouterArgs a{(int)T, (int)E, (int)top_k, sigmoid ? 1 : 0, route_norm ? 1 : 0, (float)route_scale};
  const int threads = 128;
  const unsigned blocks = (unsigned)((T * 32 + threads - 1) / threads);
  auto stream = at::cuda::getCurrentCUDAStream();
  dispatch_per_lane((int)E, [&](auto tag) {
    router_fwd_kernel<decltype(tag)::value><<<blocks, threads, 0, stream>>>(
        logits.data_ptr<float>(), bp, top.data_ptr<float>(), sel.data_ptr<int>(), counts.data_ptr<float>(), a);
  });
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  return {top, sel, counts};
}

at::Tensor moe_router_bwd(const at::Tensor& logits, const at::Tensor& sel, const at::Tensor& dtop, bool sigmoid,
                          bool route_norm, double route_scale) {
  TORCH_CHECK(logits.is_cuda() && logits.scalar_type() == at::kFloat && logits.is_contiguous());
  TORCH_CHECK(sel.scalar_type() == at::kInt && sel.is_contiguous() && dtop.scalar_type() == at::kFloat && dtop.is_contiguous());
  const int64_t T = logits.size(0), E = logits.size(1), K = sel.size(1);
  c10::cuda::CUDAGuard guard(logits.device());
  auto dl = at::empty_like(logits);
  if (T == 0) return dl;
  RouterArgs a{(int)T, (int)E, (int)K, sigmoid ? 1 : 0, route_norm ? 1 : 0, (float)route_scale};
  const int threads = 128;
  const unsigned blocks = (unsigned)((T * 32 + threads - 1) / threads);
  auto stream = at::cuda::getCurrentCUDAStream();
  dispatch_per_lane((int)E, [&](auto tag) {
    router_bwd_kernel<decltype(tag)::value><<<blocks, threads, 0, stream>>>(
        logits.data_ptr<float>(), sel.data_ptr<int>(), dtop.data_ptr<float>(), dl.data_ptr<float>(), a);
  });
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  return dl;
}

// ---------------------------------------------------------------------------------------------
// out[dest[i]] = x[i / K]   (one warp per slot, 16-byte vectors; D % 8 == 0)
__global__ void permute_rows_kernel(const __nv_bfloat16* __restrict__ x, const int* __restrict__ dest,
                                    __nv_bfloat16* __restrict__ out, int64_t slots, int K, int D) {
  const int64_t w = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (w >= slots) return;
  const int d = dest[w];
  if (d < 0) return;
  const bf16x8* src = reinterpret_cast<const bf16x8*>(x + (w / K) * D);
  bf16x8* dst = reinterpret_cast<bf16x8*>(out + (int64_t)d * D);
  for (int i = lane; i < D / 8; i += 32) dst[i] = src[i];
}

// out[t] = sum_k w[t,k] * y[dest[t,k]]  (w == nullptr: plain sum).  One warp per token.
template <bool kWeighted>
__global__ void combine_rows_kernel(const __nv_bfloat16* __restrict__ y, const int* __restrict__ dest,
                                    const float* __restrict__ wts, __nv_bfloat16* __restrict__ out, int64_t T, int K, int D) {
  const int64_t t = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (t >= T) return;
  for (int i = lane; i < D / 8; i += 32) {
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int k = 0; k < K; ++k) {
      const int d = dest[t * K + k];
      if (d < 0) continue;
      float v[8];
      unpack8(reinterpret_cast<const bf16x8*>(y + (int64_t)d * D)[i], v);
      const float wk = kWeighted ? wts[t * K + k] : 1.f;
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] += wk * v[j];
    }
    reinterpret_cast<bf16x8*>(out + t * D)[i] = pack8(acc);
  }
}

// dy[dest[t,k]] = w[t,k] * dout[t];  dw[t,k] = <dout[t], y[dest[t,k]]>.  One warp per slot.
__global__ void combine_bwd_kernel(const __nv_bfloat16* __restrict__ dout, const __nv_bfloat16* __restrict__ y,
                                   const int* __restrict__ dest, const float* __restrict__ wts,
                                   __nv_bfloat16* __restrict__ dy, float* __restrict__ dw, int64_t slots, int K, int D) {
  const int64_t s = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (s >= slots) return;
  const int d = dest[s];
  if (d < 0) {
    if (lane == 0) dw[s] = 0.f;
    return;
  }
  const float wk = wts[s];
  const bf16x8* g = reinterpret_cast<const bf16x8*>(dout + (s / K) * D);
  const bf16x8* yr = reinterpret_cast<const bf16x8*>(y + (int64_t)d * D);
  bf16x8* o = reinterpret_cast<bf16x8*>(dy + (int64_t)d * D);
  float dot = 0.f;
  for (int i = lane; i < D / 8; i += 32) {
    float gv[8], yv[8], r[8];
    unpack8(g[i], gv);
    unpack8(yr[i], yv);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      dot += gv[j] * yv[j];
      r[j] = wk * gv[j];
    }
    o[i] = pack8(r);
  }
  dot = warp_sum(dot);
  if (lane == 0) dw[s] = dot;
}

static void check_rows(const at::Tensor& t, const char* n) {
  TORCH_CHECK(t.is_cuda() && t.scalar_type() == at::kBFloat16 && t.dim() == 2 && t.is_contiguous() && t.size(1) % 8 == 0,
              "moe: ", n, " must be a contiguous bf16 [rows, D] CUDA tensor with D % 8 == 0");
}

at::Tensor moe_permute_rows(const at::Tensor& x, const at::Tensor& dest, int64_t rows) {
  check_rows(x, "x");
  TORCH_CHECK(dest.is_cuda() && dest.scalar_type() == at::kInt && dest.dim() == 2 && dest.size(0) == x.size(0) && dest.is_contiguous());
  c10::cuda::CUDAGuard guard(x.device());
  auto out = at::zeros({rows, x.size(1)}, x.options());
  const int64_t slots = dest.numel();
  if (slots == 0) return out;
  const int threads = 256;
  permute_rows_kernel<<<(unsigned)((slots * 32 + threads - 1) / threads), threads, 0, at::cuda::getCurrentCUDAStream()>>>(
      reinterpret_cast<const __nv_bfloat16*>(x.data_ptr()), dest.data_ptr<int>(),
      reinterpret_cast<__nv_bfloat16*>(out.data_ptr()), slots, (int)dest.size(1), (int)x.size(1));
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  return out;
}

at::Tensor moe_combine_rows(const at::Tensor& y, const at::Tensor& dest, const c10::optional<at::Tensor>& wts) {
  check_rows(y, "y");
  TORCH_CHECK(dest.is_cuda() && dest.scalar_type() == at::kInt && dest.dim() == 2 && dest.is_contiguous());
  c10::cuda::CUDAGuard guard(y.device());
  const int64_t T = dest.size(0);
  const int K = (int)dest.size(1), D = (int)y.size(1);
  auto out = at::empty({T, D}, y.options());
  if (T == 0) return out;
  const int threads = 256;
  const unsigned blocks = (unsigned)((T * 32 + threads - 1) / threads);
  auto stream = at::cuda::getCurrentCUDAStream();
  auto yp = reinterpret_cast<const __nv_bfloat16*>(y.data_ptr());
  auto op = reinterpret_cast<__nv_bfloat16*>(out.data_ptr());
  if (wts.has_value() && wts->defined()) {
    TORCH_CHECK(wts->is_cuda() && wts->scalar_type() == at::kFloat && wts->is_contiguous() && wts->numel() == dest.numel());
    combine_rows_kernel<true><<<blocks, threads, 0, stream>>>(yp, dest.data_ptr<int>(), wts->data_ptr<float>(), op, T, K, D);
  } else {
    combine_rows_kernel<false><<<blocks, threads, 0, stream>>>(yp, dest.data_ptr<int>(), nullptr, op, T, K, D);
  }
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  return out;
}

std::tuple<at::Tensor, at::Tensor> moe_combine_bwd(const at::Tensor& dout, const at::Tensor& y, const at::Tensor& dest,
                                                   const at::Tensor& wts) {
  check_rows(dout, "dout");
  check_rows(y, "y");
  TORCH_CHECK(dest.scalar_type() == at::kInt && dest.is_contiguous() && wts.scalar_type() == at::kFloat && wts.is_contiguous());
  c10::cuda::CUDAGuard guard(y.device());
  auto dy = at::zeros_like(y);
  auto dw = at::empty_like(wts);
  const int64_t slots = dest.numel();
  if (slots == 0) return {dy, dw};
  const int threads = 256;
  combine_bwd_kernel<<<(unsigned)((slots * 32 + threads - 1) / threads), threads, 0, at::cuda::getCurrentCUDAStream()>>>(
      reinterpret_cast<const __nv_bfloat16*>(dout.data_ptr()), reinterpret_cast<const __nv_bfloat16*>(y.data_ptr()),
      dest.data_ptr<int>(), wts.data_ptr<float>(), reinterpret_cast<__nv_bfloat16*>(dy.data_ptr()), dw.data_ptr<float>(),
      slots, (int)dest.size(1), (int)y.size(1));
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  return {dy, dw};
}

}  // namespace tb200

// =============================================================================================
// Expert-parallel exchange over NVLink symmetric memory (no NCCL all-to-all on the data path).
// Every rank knows, for each of its routing slots, the rank that hosts the chosen expert and the
// row of that rank's receive buffer (padded expert-major layout) reserved for the slot.
//   ep_scatter_rows: out_peer[dest_rank][dest_row] = (w *) x[token]       P2P stores, warp per slot
//   ep_gather_rows : out[token] = sum_k (w *) y_peer[dest_rank][dest_row]  P2P loads, warp per token;
//                    optionally keeps the gathered rows (needed for the gate-score gradient)
//   zero_pad_rows  : rows between the end of an expert's tokens and the next 128-row boundary
//   slot_dot       : dw[t, k] = <dout[t], rows[t, k]>
// Peer memory is touched with plain 16-byte loads / stores only.
namespace tb200 {

constexpr int kEpMaxPeers = 16;
struct EpPeers {
  __nv_bfloat16* p[kEpMaxPeers];
};

static EpPeers make_ep_peers(at::IntArrayRef ptrs) {
  TORCH_CHECK(ptrs.size() >= 1 && (int)ptrs.size() <= kEpMaxPeers, "ep: 1..", kEpMaxPeers, " ranks supported");
  EpPeers pp;
  for (int i = 0; i < kEpMaxPeers; ++i) pp.p[i] = nullptr;
  for (size_t i = 0; i < ptrs.size(); ++i) pp.p[i] = reinterpret_cast<__nv_bfloat16*>(static_cast<uintptr_t>(ptrs[i]));
  return pp;
}

__global__ void ep_scatter_rows_kernel(const __nv_bfloat16* __restrict__ x, const int* __restrict__ dest_rank,
                                       const int* __restrict__ dest_row, const float* __restrict__ wts, EpPeers out,
                                       int64_t slots, int K, int D) {
  const int64_t s = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (s >= slots) return;
  const int row = dest_row[s];
  if (row < 0) return;
  const bf16x8* src = reinterpret_cast<const bf16x8*>(x + (s / K) * D);
  bf16x8* dst = reinterpret_cast<bf16x8*>(out.p[dest_rank[s]] + (int64_t)row * D);
  const float w = wts == nullptr ? 1.f : wts[s];
  // four 16-byte loads in flight per lane before the (possibly remote) stores go out
  const int n = D / 8;
  for (int base = lane; base < n; base += 128) {
    bf16x8 r[4];
#pragma unroll
    for (int j = 0; j < 4; ++j)
      if (base + 32 * j < n) r[j] = src[base + 32 * j];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      if (base + 32 * j < n) {
        if (wts != nullptr) {
          float v[8];
          unpack8(r[j], v);
#pragma unroll
          for (int q = 0; q < 8; ++q) v[q] *= w;
          r[j] = pack8(v);
        }
        dst[base + 32 * j] = r[j];
      }
    }
  }
}

template <bool kWeighted>
__global__ void ep_gather_rows_kernel(EpPeers y, const int* __restrict__ dest_rank, const int* __restrict__ dest_row,
                                      const float* __restrict__ wts, __nv_bfloat16* __restrict__ out,
                                      __nv_bfloat16* __restrict__ keep, int64_t T, int K, int D) {
  const int64_t t = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (t >= T) return;
  // per 16-byte column all K rows of the token are fetched before they are summed (K independent peer loads in
  // flight instead of a load -> accumulate chain)
  constexpr int kMaxK = 8;
  for (int i = lane; i < D / 8; i += 32) {
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int k0 = 0; k0 < K; k0 += kMaxK) {
      bf16x8 raw[kMaxK];
      bool live[kMaxK];
#pragma unroll
      for (int u = 0; u < kMaxK; ++u) {
        const int k = k0 + u;
        live[u] = false;
        if (k < K) {
          const int row = dest_row[t * K + k];
          if (row >= 0) {
            live[u] = true;
            raw[u] = reinterpret_cast<const bf16x8*>(y.p[dest_rank[t * K + k]] + (int64_t)row * D)[i];
          }
        }
      }
#pragma unroll
      for (int u = 0; u < kMaxK; ++u) {
        if (!live[u]) continue;
        const int k = k0 + u;
        if (keep != nullptr) reinterpret_cast<bf16x8*>(keep + (t * K + k) * D)[i] = raw[u];
        float v[8];
        unpack8(raw[u], v);
        const float w = kWeighted ? wts[t * K + k] : 1.f;
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] += w * v[j];
      }
    }
    reinterpret_cast<bf16x8*>(out + t * D)[i] = pack8(acc);
  }
}

__global__ void zero_pad_rows_kernel(__nv_bfloat16* __restrict__ buf, const int* __restrict__ offs,
                                     const int* __restrict__ counts, int D) {
  const int e = blockIdx.x;
  const int first = offs[e] + counts[e], last = offs[e + 1];
  const int n_vec = D / 8;
  const bf16x8 zero = {};
  for (int64_t i = threadIdx.x; i < (int64_t)(last - first) * n_vec; i += blockDim.x)
    reinterpret_cast<bf16x8*>(buf + (int64_t)first * D)[i] = zero;
}

__global__ void slot_dot_kernel(const __nv_bfloat16* __restrict__ dout, const __nv_bfloat16* __restrict__ rows,
                                float* __restrict__ dw, int64_t slots, int K, int D) {
  const int64_t s = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (s >= slots) return;
  const bf16x8* g = reinterpret_cast<const bf16x8*>(dout + (s / K) * D);
  const bf16x8* r = reinterpret_cast<const bf16x8*>(rows + s * D);
  float dot = 0.f;
  for (int i = lane; i < D / 8; i += 32) {
    float a[8], b[8];
    unpack8(g[i], a);
    unpack8(r[i], b);
#pragma unroll
    for (int j = 0; j < 8; ++j) dot += a[j] * b[j];
  }
  dot = warp_sum(dot);
  if (lane == 0) dw[s] = dot;
}

static void check_slots(const at::Tensor& dest_rank, const at::Tensor& dest_row) {
  TORCH_CHECK(dest_rank.is_cuda() && dest_rank.scalar_type() == at::kInt && dest_rank.is_contiguous() && dest_rank.dim() == 2);
  TORCH_CHECK(dest_row.is_cuda() && dest_row.scalar_type() == at::kInt && dest_row.is_contiguous() &&
              dest_row.sizes() == dest_rank.sizes());
}

void ep_scatter_rows(const at::Tensor& x, const at::Tensor& dest_rank, const at::Tensor& dest_row,
                     const c10::optional<at::Tensor>& wts, at::IntArrayRef peer_ptrs) {
  check_rows(x, "x");
  check_slots(dest_rank, dest_row);
  TORCH_CHECK(dest_rank.size(0) == x.size(0));
  c10::cuda::CUDAGuard guard(x.device());
  const int64_t slots = dest_rank.numel();
  if (slots == 0) return;
  const float* wp = nullptr;
  if (wts.has_value() && wts->defined()) {
    TORCH_CHECK(wts->is_cuda() && wts->scalar_type() == at::kFloat && wts->is_contiguous() && wts->numel() == slots);
    wp = wts->data_ptr<float>();
  }
  const int threads = 256;
  ep_scatter_rows_kernel<<<(unsigned)((slots * 32 + threads - 1) / threads), threads, 0, at::cuda::getCurrentCUDAStream()>>>(
      reinterpret_cast<const __nv_bfloat16*>(x.data_ptr()), dest_rank.data_ptr<int>(), dest_row.data_ptr<int>(), wp,
      make_ep_peers(peer_ptrs), slots, (int)dest_rank.size(1), (int)x.size(1));
  C10_CUDA_KERNEL_LAUNCH_CHECK();
}

std::tuple<at::Tensor, at::Tensor> ep_gather_rows(at::IntArrayRef peer_ptrs, const at::Tensor& dest_rank,
                                                  const at::Tensor& dest_row, const c10::optional<at::Tensor>& wts,
                                                  int64_t D, bool keep_rows, const at::Tensor& like) {
  check_slots(dest_rank, dest_row);
  TORCH_CHECK(D % 8 == 0 && like.is_cuda() && like.scalar_type() == at::kBFloat16);
  c10::cuda::CUDAGuard guard(like.device());
  const int64_t T = dest_rank.size(0);
  const int K = (int)dest_rank.size(1);
  auto out = at::empty({T, D}, like.options());
  auto keep = keep_rows ? at::empty({T * K, D}, like.options()) : at::empty({0}, like.options());
  if (T == 0) return {out, keep};
  const int threads = 256;
  const unsigned blocks = (unsigned)((T * 32 + threads - 1) / threads);
  auto stream = at::cuda::getCurrentCUDAStream();
  auto kp = keep_rows ? reinterpret_cast<__nv_bfloat16*>(keep.data_ptr()) : nullptr;
  auto op = reinterpret_cast<__nv_bfloat16*>(out.data_ptr());
  const EpPeers pp = make_ep_peers(peer_ptrs);
  if (wts.has_value() && wts->defined()) {
    TORCH_CHECK(wts->is_cuda() && wts->scalar_type() == at::kFloat && wts->is_contiguous() && wts->numel() == T * K);
    ep_gather_rows_kernel<true><<<blocks, threads, 0, stream>>>(pp, dest_rank.data_ptr<int>(), dest_row.data_ptr<int>(),
                                                                 wts->data_ptr<float>(), op, kp, T, K, (int)D);
  } else {
    ep_gather_rows_kernel<false><<<blocks, threads, 0, stream>>>(pp, dest_rank.data_ptr<int>(), dest_row.data_ptr<int>(),
                                                                  nullptr, op, kp, T, K, (int)D);
  }
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  return {out, keep};
}

void moe_zero_pad_rows(at::Tensor buf, const at::Tensor& offs, const at::Tensor& counts) {
  check_rows(buf, "buf");
  TORCH_CHECK(offs.scalar_type() == at::kInt && counts.scalar_type() == at::kInt && offs.numel() == counts.numel() + 1 &&
              offs.is_contiguous() && counts.is_contiguous());
  c10::cuda::CUDAGuard guard(buf.device());
  if (counts.numel() == 0) return;
  zero_pad_rows_kernel<<<(unsigned)counts.numel(), 256, 0, at::cuda::getCurrentCUDAStream()>>>(
      reinterpret_cast<__nv_bfloat16*>(buf.data_ptr()), offs.data_ptr<int>(), counts.data_ptr<int>(), (int)buf.size(1));
  C10_CUDA_KERNEL_LAUNCH_CHECK();
}

at::Tensor moe_slot_dot(const at::Tensor& dout, const at::Tensor& rows, int64_t K) {
  check_rows(dout, "dout");
  check_rows(rows, "rows");
  TORCH_CHECK(rows.size(0) == dout.size(0) * K && rows.size(1) == dout.size(1));
  c10::cuda::CUDAGuard guard(dout.device());
  auto dw = at::empty({dout.size(0), K}, dout.options().dtype(at::kFloat));
  const int64_t slots = rows.size(0);
  if (slots > 0)
    slot_dot_kernel<<<(unsigned)((slots * 32 + 255) / 256), 256, 0, at::cuda::getCurrentCUDAStream()>>>(
        reinterpret_cast<const __nv_bfloat16*>(dout.data_ptr()), reinterpret_cast<const __nv_bfloat16*>(rows.data_ptr()),
        dw.data_ptr<float>(), slots, (int)K, (int)dout.size(1));
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  return dw;
}

// ---------------------------------------------------------------------------------------------
// Expert-parallel layout, entirely on the device (no host read, no library collective).
//
// ep_publish_counts: every rank stores its per-expert token counts into row `my_rank` of the
// symmetric count table of every peer (plain peer stores).  After a flag barrier each rank holds
// the full table counts[n_ranks][E].
//
// ep_layout: from that table each rank derives, for every routing slot (token t, choice k), the rank
// that hosts the chosen expert and the row of that rank's receive buffer reserved for the slot.  The
// receive buffer is expert-major; the rows of one expert start at a multiple of `align`, rows of lower
// source ranks come first, and within a source rank the slots keep token order (stable, hence
// deterministic).  One block per expert: it recomputes the prefix of padded group sizes of the owner
// rank, then walks over all slots in order with a block-wide exclusive scan of "slot chose this
// expert".  A slot whose row would fall outside the static capacity gets row -1 (the scatter / gather
// kernels skip it) and kStatusEpOverflow is set in the status word.
constexpr int kLayoutThreads = 1024;
constexpr int kLayoutPerThread = 8;
constexpr int kStatusEpOverflow = 1 << 3;

__global__ void ep_publish_counts_kernel(const float* __restrict__ counts, EpPeers tables, int n_ranks, int my_rank, int E) {
  for (int i = threadIdx.x; i < n_ranks * E; i += blockDim.x) {
    const int q = i / E, e = i % E;
    reinterpret_cast<int*>(tables.p[q])[my_rank * E + e] = (int)counts[e];
  }
}

__global__ void __launch_bounds__(kLayoutThreads)
ep_layout_kernel(const int* __restrict__ selected, const int* __restrict__ table, int n_ranks, int my_rank, int E,
                 int64_t slots, int cap, int align, int* __restrict__ dest_rank, int* __restrict__ dest_row,
                 int* __restrict__ my_offs, int* __restrict__ my_counts, int* __restrict__ status) {
  const int e = blockIdx.x;
  const int El = E / n_ranks;
  const int owner = e / El, e_loc = e % El;
  __shared__ int s_warp[kLayoutThreads / 32];
  __shared__ int s_base, s_running, s_limit;
  if (threadIdx.x == 0) {
    // first row of expert e in the owner's buffer, then the rows of lower source ranks
    int start = 0;
    for (int j = 0; j < e_loc; ++j) {
      int tot = 0;
      for (int r = 0; r < n_ranks; ++r) tot += table[r * E + owner * El + j];
      start += (tot + align - 1) / align * align;
    }
    int before = 0;
    for (int r = 0; r < my_rank; ++r) before += table[r * E + e];
    s_base = start + before;
    s_running = 0;
    s_limit = cap;
    if (owner == my_rank) {
      int tot = 0;
      for (int r = 0; r < n_ranks; ++r) tot += table[r * E + e];
      my_offs[e_loc] = start;
      my_counts[e_loc] = tot;
      if (e_loc == El - 1) {
        const int end = start + (tot + align - 1) / align * align;
        my_offs[El] = min(end, cap / align * align);
        if (end > cap) atomicOr(status, kStatusEpOverflow);
      }
    }
  }
  __syncthreads();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int64_t chunk = 0; chunk < slots; chunk += (int64_t)kLayoutThreads * kLayoutPerThread) {
    const int64_t i0 = chunk + (int64_t)threadIdx.x * kLayoutPerThread;
    int hit[kLayoutPerThread];
    int mine = 0;
#pragma unroll
    for (int u = 0; u < kLayoutPerThread; ++u) {
      hit[u] = (i0 + u < slots && selected[i0 + u] == e) ? 1 : 0;
      mine += hit[u];
    }
    // exclusive scan of `mine` over the block
    int incl = mine;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int v = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += v;
    }
    if (lane == 31) s_warp[warp] = incl;
    __syncthreads();
    if (warp == 0) {
      int w = s_warp[lane];
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int v = __shfl_up_sync(0xffffffffu, w, o);
        if (lane >= o) w += v;
      }
      s_warp[lane] = w;   // inclusive scan of the warp totals
    }
    __syncthreads();
    const int running = s_running;
    int pos = s_base + running + (warp > 0 ? s_warp[warp - 1] : 0) + incl - mine;
#pragma unroll
    for (int u = 0; u < kLayoutPerThread; ++u) {
      if (hit[u]) {
        const bool fits = pos < s_limit;
        dest_rank[i0 + u] = owner;
        dest_row[i0 + u] = fits ? pos : -1;
        if (!fits) atomicOr(status, kStatusEpOverflow);
        ++pos;
      }
    }
    __syncthreads();
    if (threadIdx.x == 0) s_running = running + s_warp[kLayoutThreads / 32 - 1];
    __syncthreads();
  }
}

void ep_publish_counts(const at::Tensor& counts, at::IntArrayRef table_ptrs, int64_t my_rank) {
  TORCH_CHECK(counts.is_cuda() && counts.scalar_type() == at::kFloat && counts.is_contiguous());
  c10::cuda::CUDAGuard guard(counts.device());
  const EpPeers pp = make_ep_peers(table_ptrs);
  ep_publish_counts_kernel<<<1, 256, 0, at::cuda::getCurrentCUDAStream()>>>(counts.data_ptr<float>(), pp, (int)table_ptrs.size(),
                                                                             (int)my_rank, (int)counts.numel());
  C10_CUDA_KERNEL_LAUNCH_CHECK();
}

// selected [T, K] int32, table [n_ranks, E] int32 (this rank's copy) -> (dest_rank [T, K], dest_row [T, K],
// my_offs [E / n_ranks + 1], my_counts [E / n_ranks]); `status` collects kStatusEpOverflow.
std::tuple<at::Tensor, at::Tensor, at::Tensor, at::Tensor> ep_layout(const at::Tensor& selected, const at::Tensor& table,
                                                                     int64_t my_rank, int64_t cap, int64_t align,
                                                                     at::Tensor status) {
  TORCH_CHECK(selected.is_cuda() && selected.scalar_type() == at::kInt && selected.is_contiguous() && selected.dim() == 2);
  TORCH_CHECK(table.is_cuda() && table.scalar_type() == at::kInt && table.is_contiguous() && table.dim() == 2);
  TORCH_CHECK(status.is_cuda() && status.scalar_type() == at::kInt && status.numel() >= 1);
  const int n = (int)table.size(0), E = (int)table.size(1);
  TORCH_CHECK(E % n == 0 && my_rank >= 0 && my_rank < n && align > 0 && cap >= align);
  c10::cuda::CUDAGuard guard(selected.device());
  auto iopt = selected.options();
  auto dest_rank = at::empty_like(selected);
  auto dest_row = at::empty_like(selected);
  auto my_offs = at::zeros({E / n + 1}, iopt);
  auto my_counts = at::zeros({E / n}, iopt);
  if (selected.numel() > 0 || true)
    ep_layout_kernel<<<E, kLayoutThreads, 0, at::cuda::getCurrentCUDAStream()>>>(
        selected.data_ptr<int>(), table.data_ptr<int>(), n, (int)my_rank, E, selected.numel(), (int)cap, (int)align,
        dest_rank.data_ptr<int>(), dest_row.data_ptr<int>(), my_offs.data_ptr<int>(), my_counts.data_ptr<int>(),
        status.data_ptr<int>());
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  return {dest_rank, dest_row, my_offs, my_counts};
}

}  // namespace tb200
