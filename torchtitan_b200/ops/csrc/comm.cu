// In-kernel NVLink communication over symmetric memory (peer pointers of one NVSwitch domain).
//
//  * symm_barrier: every rank publishes an epoch number into each peer's flag array and waits
//    for all peers' epochs.  Waits are bounded: after `max_cycles` the kernel records
//    kStatusWaitTimedOut in the caller's status word and returns, it never traps or spins
//    forever.
//  * reduce_scatter_pull: each rank pulls its 1/N slice of every peer's gradient buffer with
//    16-byte peer loads, accumulates in fp32 and writes (or adds into) its fp32 gradient shard.
//    The wire format is the gradient dtype (bf16): half the bytes of an fp32 reduce-scatter and
//    no cast / copy-in pass.
//  * adamw_allgather: the sharded AdamW update that also writes the refreshed low-precision
//    weights into every peer's parameter buffer with peer stores, i.e. the parameter
//    all-gather happens inside the optimizer kernel.
//
// Peer memory is only touched with plain ld/st.global (no TMA, no multicast loads).
#include <cstdlib>
#include <ATen/ATen.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>

#include "common.cuh"

namespace tb200 {

constexpr int kMaxPeers = 16;

struct PeerPtrs {
  void* p[kMaxPeers];
};

static PeerPtrs make_peers(at::IntArrayRef ptrs) {
  TORCH_CHECK(ptrs.size() >= 1 && (int)ptrs.size() <= kMaxPeers, "tb200: 1..", kMaxPeers, " peers supported");
  PeerPtrs pp;
  for (int i = 0; i < kMaxPeers; ++i) pp.p[i] = nullptr;
  for (size_t i = 0; i < ptrs.size(); ++i) pp.p[i] = reinterpret_cast<void*>(static_cast<uintptr_t>(ptrs[i]));
  return pp;
}

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// flags[q] on rank r holds the latest epoch published by rank q.  The epoch is a device-side
// counter that the kernel itself advances: every rank runs the same sequence of barriers on an
// arena, so the counters stay equal across ranks, and a barrier replayed from a CUDA graph
// publishes a fresh epoch on every replay (a host-side counter would be frozen into the graph).
// `bump`, when given, is a second counter advanced by one in the same launch (the fused
// all-gather GEMM that follows reads it as its own epoch).
__global__ void symm_barrier_kernel(PeerPtrs flags, int nranks, int my_rank, uint32_t* epoch_counter, uint32_t* bump,
                                    int* status, long long max_cycles) {
  __shared__ uint32_t s_epoch;
  const int t = threadIdx.x;
  if (t == 0) {
    s_epoch = atomicAdd(epoch_counter, 1u) + 1u;
    if (bump != nullptr) atomicAdd(bump, 1u);
  }
  __syncthreads();
  const uint32_t epoch = s_epoch;
  if (t >= nranks) return;
  __threadfence_system();
  st_release_sys(reinterpret_cast<uint32_t*>(flags.p[t]) + my_rank, epoch);
  const uint32_t* mine = reinterpret_cast<const uint32_t*>(flags.p[my_rank]) + t;
  const long long start = clock64();
  while (true) {
    const uint32_t v = ld_acquire_sys(mine);
    if ((int32_t)(v - epoch) >= 0) break;
    if (clock64() - start > max_cycles) {
      atomicOr(status, kStatusWaitTimedOut);
      break;
    }
    __nanosleep(64);
  }
}

void symm_barrier(at::IntArrayRef flag_ptrs, int64_t my_rank, at::Tensor epoch, at::Tensor status, int64_t max_cycles,
                  const c10::optional<at::Tensor>& bump) {
  TORCH_CHECK(status.is_cuda() && status.scalar_type() == at::kInt && status.numel() >= 1);
  TORCH_CHECK(epoch.is_cuda() && epoch.scalar_type() == at::kInt && epoch.numel() == 1, "symm_barrier: epoch is an int32[1] device tensor");
  TORCH_CHECK((int)flag_ptrs.size() <= 32, "symm_barrier: at most 32 ranks");
  uint32_t* bp = nullptr;
  if (bump.has_value() && bump->defined()) {
    TORCH_CHECK(bump->is_cuda() && bump->scalar_type() == at::kInt && bump->numel() == 1);
    bp = reinterpret_cast<uint32_t*>(bump->data_ptr<int>());
  }
  c10::cuda::CUDAGuard guard(status.device());
  const PeerPtrs pp = make_peers(flag_ptrs);
  auto stream = at::cuda::getCurrentCUDAStream();
  symm_barrier_kernel<<<1, 32, 0, stream>>>(pp, (int)flag_ptrs.size(), (int)my_rank,
                                            reinterpret_cast<uint32_t*>(epoch.data_ptr<int>()), bp, status.data_ptr<int>(),
                                            (long long)max_cycles);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
}

template <typename T>
__device__ __forceinline__ void ld8(const T* p, float (&f)[8]);
template <>
__device__ __forceinline__ void ld8<float>(const float* p, float (&f)[8]) {
  const float4 a = *reinterpret_cast<const float4*>(p);
  const float4 b = *reinterpret_cast<const float4*>(p + 4);
  f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
}
template <>
__device__ __forceinline__ void ld8<__nv_bfloat16>(const __nv_bfloat16* p, float (&f)[8]) {
  unpack8(*reinterpret_cast<const bf16x8*>(p), f);
}
template <typename T>
__device__ __forceinline__ void st8(T* p, const float (&f)[8]);
template <>
__device__ __forceinline__ void st8<float>(float* p, const float (&f)[8]) {
  *reinterpret_cast<float4*>(p) = make_float4(f[0], f[1], f[2], f[3]);
  *reinterpret_cast<float4*>(p + 4) = make_float4(f[4], f[5], f[6], f[7]);
}
template <>
__device__ __forceinline__ void st8<__nv_bfloat16>(__nv_bfloat16* p, const float (&f)[8]) {
  *reinterpret_cast<bf16x8*>(p) = pack8(f);
}

// out[i] (+)= sum_q peers[q][offset + i], i in [0, n); n and offset multiples of 8.
template <typename G, int NR>
__global__ void __launch_bounds__(256) reduce_scatter_pull_kernel(PeerPtrs peers, int nranks_rt, int my_rank,
                                                                  int64_t offset, int64_t nvec, float* __restrict__ out,
                                                                  int accumulate) {
  const int nranks = NR > 0 ? NR : nranks_rt;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += (int64_t)gridDim.x * blockDim.x) {
    float acc[8];
    if (accumulate) {
      ld8<float>(out + i * 8, acc);
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] = 0.f;
    }
    if (NR > 0) {
      float f[NR > 0 ? NR : 1][8];
#pragma unroll
      for (int q = 0; q < NR; ++q) {
        const int src = (my_rank + q) % NR;  // own memory first, then rotate so links are spread
        ld8<G>(reinterpret_cast<const G*>(peers.p[src]) + offset + i * 8, f[q]);
      }
#pragma unroll
      for (int q = 0; q < NR; ++q)
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] += f[q][j];
    } else {
      for (int q = 0; q < nranks; ++q) {
        const int src = (my_rank + q) % nranks;
        float f[8];
        ld8<G>(reinterpret_cast<const G*>(peers.p[src]) + offset + i * 8, f);
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] += f[j];
      }
    }
    st8<float>(out + i * 8, acc);
  }
}

// Thread blocks per SM of the communication kernels that run on a side stream next to the GEMMs.  More blocks keep
// more peer loads in flight; fewer leave more issue slots and memory bandwidth to the compute stream.  The environment
// variable TB200_COMM_CTAS_PER_SM overrides the per-kernel default (read once).
static int comm_ctas_per_sm(int dflt) {
  static const int env = [] {
    const char* e = std::getenv("TB200_COMM_CTAS_PER_SM");
    const int v = e ? std::atoi(e) : 0;
    return v > 0 && v <= 32 ? v : 0;
  }();
  return env ? env : dflt;
}

void reduce_scatter_pull(at::IntArrayRef grad_ptrs, int64_t my_rank, int64_t offset, at::Tensor out, bool grad_is_bf16,
                         bool accumulate) {
  TORCH_CHECK(out.is_cuda() && out.scalar_type() == at::kFloat && out.is_contiguous());
  const int64_t n = out.numel();
  TORCH_CHECK(n % 8 == 0 && offset % 8 == 0, "reduce_scatter_pull: shard size and offset must be multiples of 8");
  if (n == 0) return;
  c10::cuda::CUDAGuard guard(out.device());
  const PeerPtrs pp = make_peers(grad_ptrs);
  const int nr = (int)grad_ptrs.size();
  auto stream = at::cuda::getCurrentCUDAStream();
  const int64_t nvec = n / 8;
  const int grid = (int)std::max<int64_t>(1, std::min<int64_t>((nvec + 255) / 256, (int64_t)num_sms() * comm_ctas_per_sm(8)));
  float* op = out.data_ptr<float>();
#define TB_RS(G, NR) \
  reduce_scatter_pull_kernel<G, NR><<<grid, 256, 0, stream>>>(pp, nr, (int)my_rank, offset, nvec, op, accumulate ? 1 : 0)
  if (grad_is_bf16) {
    using G = __nv_bfloat16;
    if (nr == 2) TB_RS(G, 2);
    else if (nr == 4) TB_RS(G, 4);
    else if (nr == 8) TB_RS(G, 8);
    else TB_RS(G, 0);
  } else {
    using G = float;
    if (nr == 2) TB_RS(G, 2);
    else if (nr == 4) TB_RS(G, 4);
    else if (nr == 8) TB_RS(G, 8);
    else TB_RS(G, 0);
  }
#undef TB_RS
  C10_CUDA_KERNEL_LAUNCH_CHECK();
}

// out[q * n16 + i] = peers[q][i] for every rank q (16-byte units): an all-gather by peer loads.
// Rank order is rotated per block so that the ranks do not all read the same peer at once.
__global__ void __launch_bounds__(256) all_gather_pull_kernel(PeerPtrs peers, int nranks, int my_rank, int64_t n16,
                                                              uint4* __restrict__ out) {
  const int64_t total = n16 * nranks;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int slot = (int)(i / n16);
    const int64_t off = i - (int64_t)slot * n16;
    const int q = (my_rank + slot) % nranks;
    out[(int64_t)q * n16 + off] = reinterpret_cast<const uint4*>(peers.p[q])[off];
  }
}

// Gather `nbytes` (a multiple of 16) from the same symmetric buffer of every rank into `out`
// ([nranks * nbytes], rank-major).
void all_gather_pull(at::IntArrayRef src_ptrs, int64_t my_rank, int64_t nbytes, at::Tensor out) {
  TORCH_CHECK(out.is_cuda() && out.is_contiguous());
  const int nr = (int)src_ptrs.size();
  TORCH_CHECK(nbytes % 16 == 0 && (int64_t)out.numel() * out.element_size() == nbytes * nr,
              "all_gather_pull: the output must hold nranks * nbytes and nbytes must be a multiple of 16");
  TORCH_CHECK((reinterpret_cast<uintptr_t>(out.data_ptr()) & 15u) == 0, "all_gather_pull: unaligned output");
  if (nbytes == 0) return;
  c10::cuda::CUDAGuard guard(out.device());
  const PeerPtrs pp = make_peers(src_ptrs);
  const int64_t n16 = nbytes / 16;
  const int grid = (int)std::max<int64_t>(1, std::min<int64_t>((n16 * nr + 255) / 256, (int64_t)num_sms() * 8));
  all_gather_pull_kernel<<<grid, 256, 0, at::cuda::getCurrentCUDAStream()>>>(pp, nr, (int)my_rank, n16,
                                                                              reinterpret_cast<uint4*>(out.data_ptr()));
  C10_CUDA_KERNEL_LAUNCH_CHECK();
}

// 8 elements to a multicast address (multimem.st: the switch replicates the store to all ranks).
__device__ __forceinline__ void mc_st16(void* p, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};"
               ::"l"(p), "f"(__uint_as_float(a)), "f"(__uint_as_float(b)), "f"(__uint_as_float(c)), "f"(__uint_as_float(d))
               : "memory");
}
template <typename T>
__device__ __forceinline__ void mc_st8(T* p, const float (&f)[8]);
template <>
__device__ __forceinline__ void mc_st8<float>(float* p, const float (&f)[8]) {
  mc_st16(p, __float_as_uint(f[0]), __float_as_uint(f[1]), __float_as_uint(f[2]), __float_as_uint(f[3]));
  mc_st16(p + 4, __float_as_uint(f[4]), __float_as_uint(f[5]), __float_as_uint(f[6]), __float_as_uint(f[7]));
}
template <>
__device__ __forceinline__ void mc_st8<__nv_bfloat16>(__nv_bfloat16* p, const float (&f)[8]) {
  uint32_t w[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    __nv_bfloat162 h = __floats2bfloat162_rn(f[2 * j], f[2 * j + 1]);
    w[j] = *reinterpret_cast<uint32_t*>(&h);
  }
  mc_st16(p, w[0], w[1], w[2], w[3]);
}

// AdamW on this rank's shard; the updated low-precision weights are stored into every peer's
// parameter buffer at `offset` (the all-gather).
template <typename G, typename S, typename P>
__global__ void __launch_bounds__(256) adamw_allgather_kernel(float* __restrict__ master, const G* __restrict__ grad,
                                                              S* __restrict__ m, S* __restrict__ v, PeerPtrs params,
                                                              P* __restrict__ mc_params, int nranks, int my_rank, int64_t offset,
                                                              const float* __restrict__ grad_scale, int64_t nvec,
                                                              float lr, float beta1, float beta2, float eps, float wd,
                                                              float bc1, float bc2_sqrt) {
  const float gs = *grad_scale;
  if (!isfinite(gs)) return;
  const float step_size = lr / bc1;
  const float decay = 1.f - lr * wd;
  const float inv_bc2 = 1.f / bc2_sqrt;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t o = i * 8;
    float g[8], mm[8], vv[8], p[8];
    ld8<G>(grad + o, g);
    ld8<S>(m + o, mm);
    ld8<S>(v + o, vv);
    ld8<float>(master + o, p);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float gj = g[j] * gs;
      mm[j] = beta1 * mm[j] + (1.f - beta1) * gj;
      vv[j] = beta2 * vv[j] + (1.f - beta2) * gj * gj;
      const float denom = sqrtf(vv[j]) * inv_bc2 + eps;
      p[j] = p[j] * decay - step_size * (mm[j] / denom);
    }
    st8<float>(master + o, p);
    st8<S>(m + o, mm);
    st8<S>(v + o, vv);
    if (mc_params != nullptr) {
      // one store through the NVSwitch multicast object reaches the buffer of every rank (this one included)
      mc_st8<P>(mc_params + offset + o, p);
    } else {
      for (int q = 0; q < nranks; ++q) {
        const int dst = (my_rank + q) % nranks;
        st8<P>(reinterpret_cast<P*>(params.p[dst]) + offset + o, p);
      }
    }
  }
}

void adamw_allgather_(at::Tensor master, const at::Tensor& grad, at::Tensor exp_avg, at::Tensor exp_avg_sq,
                      at::IntArrayRef param_ptrs, int64_t my_rank, int64_t offset, bool param_is_bf16,
                      int64_t multicast_ptr, const at::Tensor& grad_scale, double lr, double beta1, double beta2, double eps,
                      double weight_decay, double bc1, double bc2) {
  TORCH_CHECK(master.is_cuda() && master.scalar_type() == at::kFloat && master.is_contiguous());
  const int64_t n = master.numel();
  TORCH_CHECK(n % 8 == 0 && offset % 8 == 0, "adamw_allgather_: segment size and offset must be multiples of 8");
  TORCH_CHECK(grad.numel() == n && exp_avg.numel() == n && exp_avg_sq.numel() == n);
  TORCH_CHECK(grad.scalar_type() == at::kFloat, "adamw_allgather_: reduced gradients are fp32");
  TORCH_CHECK(exp_avg.scalar_type() == exp_avg_sq.scalar_type());
  if (n == 0) return;
  c10::cuda::CUDAGuard guard(master.device());
  const PeerPtrs pp = make_peers(param_ptrs);
  const int nr = (int)param_ptrs.size();
  auto stream = at::cuda::getCurrentCUDAStream();
  const int64_t nvec = n / 8;
  const int grid = (int)std::max<int64_t>(1, std::min<int64_t>((nvec + 255) / 256, (int64_t)num_sms() * comm_ctas_per_sm(16)));
  const bool sb = exp_avg.scalar_type() == at::kBFloat16;
  TORCH_CHECK(sb || exp_avg.scalar_type() == at::kFloat);
#define TB_AG(S, P)                                                                                             \
  adamw_allgather_kernel<float, S, P><<<grid, 256, 0, stream>>>(                                                  \
      master.data_ptr<float>(), grad.data_ptr<float>(), reinterpret_cast<S*>(exp_avg.data_ptr()),                 \
      reinterpret_cast<S*>(exp_avg_sq.data_ptr()), pp, reinterpret_cast<P*>(multicast_ptr), nr, (int)my_rank, offset, \
      grad_scale.data_ptr<float>(), nvec,                                                                          \
      (float)lr, (float)beta1, (float)beta2, (float)eps, (float)weight_decay, (float)bc1, sqrtf((float)bc2))
  using bf16 = __nv_bfloat16;
  if (sb && param_is_bf16) TB_AG(bf16, bf16);
  else if (sb) TB_AG(bf16, float);
  else if (param_is_bf16) TB_AG(float, bf16);
  else TB_AG(float, float);
#undef TB_AG
  C10_CUDA_KERNEL_LAUNCH_CHECK();
}

}  // namespace tb200
