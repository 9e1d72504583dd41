// Flash attention for head dimension 128 on the 5th-generation tensor cores.
//
// Forward.  One CTA owns a block of 128 query rows for up to two query heads that share one
// key/value head (grouped-query attention), so each K/V tile brought in by TMA serves both.
// Per K/V tile of 128 rows and per head ("slot"):
//     S = Q . K^T          tcgen05.mma, operands in shared memory, S (fp32) in tensor memory
//     P = exp2(S - m)      softmax warps: one thread per query row reads its row of S with
//                          tcgen05.ld, writes bf16 P back over S with tcgen05.st
//     O += P . V           tcgen05.mma with the A operand (P) read from tensor memory
// The two slots alternate on the tensor pipe, so the softmax of one overlaps the MMAs of the
// other.  The running maximum is only raised when it grew by more than 2^8 (the accumulator in
// tensor memory is rescaled in place at that point), which removes most rescaling passes.
//
//   warp 0       TMA producer (Q once; K and V tiles through two-stage rings)
//   warp 1       TMEM allocation, MMA issue (one elected lane)
//   warps 2..5   softmax + epilogue of slot 0 (TMEM lane quarter = warp % 4)
//   warps 6..9   softmax + epilogue of slot 1
// Tensor memory (512 columns): slot s uses columns [256 s, 256 s + 128) for S / P and
// [256 s + 128, 256 s + 256) for O.
//
// Masking: causal with an offset (query row i sees keys <= i + offset), an optional first
// visible key per query row (packed documents), and the end of the key sequence.
//
// All mbarrier waits are bounded; on a timeout every role leaves its loop, TMEM is released and
// kStatusWaitTimedOut is set in the status word.  TMA loads are plain tile loads.
#include <ATen/ATen.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <cuda.h>

#include "common.cuh"
#include "tc.cuh"

namespace tb200 {
namespace flash {

using namespace tc;

constexpr int kD = 128;          // head dimension
constexpr int kBM = 128;         // query rows per CTA
constexpr int kBN = 128;         // key rows per tile
constexpr int kThreadsFwd = 320;
constexpr uint32_t kTileBytes = 128 * kD * 2;   // 32 KB: one 128 x 128 bf16 tile (two 64-column swizzled halves)
constexpr uint32_t kHalfBytes = kTileBytes / 2;
constexpr float kRescaleThreshold = 8.0f;       // in log2 units

struct FwdParams {
  int Tq, Tk, Hq, Hkv;
  int causal;
  int causal_offset;       // query row i sees keys j <= i + causal_offset
  int slots;               // query heads per CTA (1 or 2)
  int ctas_per_kv_head;    // group / slots
  float scale_log2;        // softmax scale * log2(e)
  const int* kv_first;     // [Tq] first visible key per query row, or nullptr
  float* lse;              // [Hq, Tq] natural-log sum-exp of the scaled scores
  int* status;
};

__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t* r) {
  uint32_t a[16], b[16];
#pragma unroll
  for (int i = 0; i < 16; ++i) { a[i] = r[i]; b[i] = r[16 + i]; }
  tmem_st16(taddr, a);
  tmem_st16(taddr + 16, b);
}

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&h);
}

__global__ void __launch_bounds__(kThreadsFwd, 1)
flash_fwd_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                 const __grid_constant__ CUtensorMap tmap_v, const __grid_constant__ CUtensorMap tmap_o,
                 const FwdParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* gen_base = smem_raw + (base - raw);
  // shared memory: Q[2 slots] | K ring[2] | V ring[2] | barriers
  const uint32_t q_smem = base;
  const uint32_t k_smem = base + 2 * kTileBytes;
  const uint32_t v_smem = base + 4 * kTileBytes;
  const uint32_t bar_base = base + 6 * kTileBytes;
  enum { Q_FULL = 0, K_FULL = 1, K_EMPTY = 3, V_FULL = 5, V_EMPTY = 7, S_FULL = 9, P_READY = 11, O_FULL = 13, O_STAGED = 14, NBAR = 16 };
  auto bar = [&](int i) { return bar_base + 8u * i; };
  uint32_t* tmem_ptr_smem = reinterpret_cast<uint32_t*>(gen_base + 6 * kTileBytes + 8 * NBAR);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_ptr_smem + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  // ---- work assignment: longest query blocks first
  const int num_q_tiles = (p.Tq + kBM - 1) / kBM;
  const int per_tile = p.Hkv * p.ctas_per_kv_head;
  const int q_tile = num_q_tiles - 1 - (int)blockIdx.x / per_tile;
  const int rem = (int)blockIdx.x % per_tile;
  const int kv_head = rem / p.ctas_per_kv_head;
  const int group = p.Hq / p.Hkv;
  const int head0 = kv_head * group + (rem % p.ctas_per_kv_head) * p.slots;
  const int q0 = q_tile * kBM;
  // key tile range [j_lo, j_hi]
  const int num_k_tiles = (p.Tk + kBN - 1) / kBN;
  int j_hi = num_k_tiles - 1;
  if (p.causal) j_hi = min(j_hi, (min(q0 + kBM - 1, p.Tq - 1) + p.causal_offset) / kBN);
  int j_lo = 0;
  if (p.kv_first != nullptr) j_lo = max(0, p.kv_first[q0]) / kBN;   // kv_first is non-decreasing
  const int n_tiles = j_hi - j_lo + 1;                                // may be <= 0: nothing visible

  if (threadIdx.x == 0) {
    mbar_init(bar(Q_FULL), 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(bar(K_FULL + s), 1);
      mbar_init(bar(K_EMPTY + s), 1);
      mbar_init(bar(V_FULL + s), 1);
      mbar_init(bar(V_EMPTY + s), 1);
      mbar_init(bar(S_FULL + s), 1);
      mbar_init(bar(P_READY + s), 128);
      mbar_init(bar(O_STAGED + s), 128);
    }
    mbar_init(bar(O_FULL), 1);
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmap_q);
    tma_prefetch_desc(&tmap_k);
    tma_prefetch_desc(&tmap_v);
    tma_prefetch_desc(&tmap_o);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_ptr_smem), 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_ptr_smem;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0 && n_tiles > 0) {
      mbar_expect_tx(bar(Q_FULL), (uint32_t)p.slots * kTileBytes);
      for (int s = 0; s < p.slots; ++s)
        for (int h = 0; h < 2; ++h)
          tma_load_3d(q_smem + s * kTileBytes + h * kHalfBytes, &tmap_q, bar(Q_FULL), h * 64, head0 + s, q0);
      for (int i = 0; i < n_tiles; ++i) {
        const int st = i & 1;
        const uint32_t parity = ((i >> 1) & 1u) ^ 1u;
        const int k0 = (j_lo + i) * kBN;
        if (!mbar_wait(bar(K_EMPTY + st), parity, abort_flag)) break;
        mbar_expect_tx(bar(K_FULL + st), kTileBytes);
        for (int h = 0; h < 2; ++h)
          tma_load_3d(k_smem + st * kTileBytes + h * kHalfBytes, &tmap_k, bar(K_FULL + st), h * 64, kv_head, k0);
        if (!mbar_wait(bar(V_EMPTY + st), parity, abort_flag)) break;
        mbar_expect_tx(bar(V_FULL + st), kTileBytes);
        for (int h = 0; h < 2; ++h)
          tma_load_3d(v_smem + st * kTileBytes + h * kHalfBytes, &tmap_v, bar(V_FULL + st), h * 64, kv_head, k0);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0 && n_tiles > 0) {
      const uint32_t idesc_s = make_idesc(false, false, kBM, kBN);   // Q, K both K-major (head dim contiguous)
      const uint32_t idesc_pv = make_idesc(false, true, kBM, kD);    // V is [keys, head dim]: MN-major B
      auto issue_s = [&](int slot, int st) {
        const uint32_t qa = q_smem + slot * kTileBytes, ka = k_smem + st * kTileBytes;
#pragma unroll
        for (int k = 0; k < kD / 16; ++k) {
          const uint32_t off = (uint32_t)(k >> 2) * kHalfBytes + (uint32_t)(k & 3) * 32u;
          umma_bf16<1>(tmem_base + slot * 256, make_desc(qa + off, 16, 1024), make_desc(ka + off, 16, 1024), idesc_s,
                       k != 0 ? 1u : 0u);
        }
      };
      auto issue_pv = [&](int slot, int st, bool accumulate) {
        const uint32_t va = v_smem + st * kTileBytes;
#pragma unroll
        for (int k = 0; k < kBN / 16; ++k)   // 16 keys per step: 8 packed columns of P, 16 rows (2048 B) of V
          umma_bf16_ts(tmem_base + slot * 256 + 128, tmem_base + slot * 256 + k * 8,
                       make_desc(va + k * 2048, kHalfBytes, 1024), idesc_pv, (accumulate || k != 0) ? 1u : 0u);
      };
      bool ok = mbar_wait(bar(Q_FULL), 0, abort_flag) && mbar_wait(bar(K_FULL), 0, abort_flag);
      if (ok) {
        tc_fence_after();
        for (int s = 0; s < p.slots; ++s) {
          issue_s(s, 0);
          umma_commit(bar(S_FULL + s));
        }
        umma_commit(bar(K_EMPTY));
      }
      for (int i = 0; i < n_tiles && ok; ++i) {
        const int st = i & 1;
        if (!mbar_wait(bar(V_FULL + st), (i >> 1) & 1u, abort_flag)) { ok = false; break; }
        for (int s = 0; s < p.slots && ok; ++s) {
          if (!mbar_wait(bar(P_READY + s), i & 1u, abort_flag)) { ok = false; break; }
          tc_fence_after();
          issue_pv(s, st, i > 0);
          if (s == p.slots - 1) umma_commit(bar(V_EMPTY + st));
          if (i + 1 < n_tiles) {
            const int st1 = (i + 1) & 1;
            if (s == 0 && !mbar_wait(bar(K_FULL + st1), ((i + 1) >> 1) & 1u, abort_flag)) { ok = false; break; }
            tc_fence_after();
            issue_s(s, st1);
            umma_commit(bar(S_FULL + s));
            if (s == p.slots - 1) umma_commit(bar(K_EMPTY + st1));
          }
        }
      }
      if (ok) umma_commit(bar(O_FULL));
    }
  } else {
    // ------------------------------------------------------------------ softmax + epilogue
    const int slot = (warp - 2) >> 2;
    const int quarter = warp & 3;
    if (slot < p.slots) {
      const int row_in_tile = quarter * 32 + lane;
      const int row = q0 + row_in_tile;
      const uint32_t s_t = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(slot * 256);
      const uint32_t o_t = s_t + 128;
      const int lo = p.kv_first != nullptr ? p.kv_first[min(row, p.Tq - 1)] : 0;          // first visible key
      const int hi = min(p.Tk - 1, p.causal ? row + p.causal_offset : p.Tk - 1);           // last visible key
      float m_used = -INFINITY, l = 0.f;
      bool ok = true;
      for (int i = 0; i < n_tiles; ++i) {
        if (!mbar_wait(bar(S_FULL + slot), i & 1u, abort_flag)) { ok = false; break; }
        tc_fence_after();
        uint32_t r[4][32];
#pragma unroll
        for (int c = 0; c < 4; ++c) tmem_ld32(s_t + c * 32, r[c]);
        tmem_ld_wait();
        const int c0 = (j_lo + i) * kBN;
        const bool edge = (c0 + kBN - 1 > hi) || (c0 < lo);
        float m_tile = -INFINITY;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
#pragma unroll
          for (int e = 0; e < 32; ++e) {
            float x = __uint_as_float(r[c][e]) * p.scale_log2;
            if (edge) {
              const int col = c0 + c * 32 + e;
              if (col > hi || col < lo) x = -INFINITY;
            }
            r[c][e] = __float_as_uint(x);
            m_tile = fmaxf(m_tile, x);
          }
        }
        const float m_new = fmaxf(m_used, m_tile);
        if (__any_sync(0xffffffffu, m_new > m_used + kRescaleThreshold)) {
          // every row of this warp moves to its own new maximum; O and l are rescaled
          const float alpha = (m_used == -INFINITY) ? 0.f : exp2f(m_used - m_new);
          l *= alpha;
          if (i > 0) {
#pragma unroll 1
            for (int c = 0; c < 4; ++c) {
              uint32_t o[32];
              tmem_ld32(o_t + c * 32, o);
              tmem_ld_wait();
#pragma unroll
              for (int e = 0; e < 32; ++e) o[e] = __float_as_uint(__uint_as_float(o[e]) * alpha);
              tmem_st32(o_t + c * 32, o);
            }
          }
          m_used = m_new;
        }
        const float m_eff = (m_used == -INFINITY) ? 0.f : m_used;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint32_t pk[16];
#pragma unroll
          for (int e = 0; e < 16; ++e) {
            const float p0 = exp2f(__uint_as_float(r[c][2 * e]) - m_eff);
            const float p1 = exp2f(__uint_as_float(r[c][2 * e + 1]) - m_eff);
            l += p0 + p1;
            pk[e] = pack_bf16(p0, p1);
          }
          tmem_st16(s_t + c * 16, pk);
        }
        tmem_st_wait();
        tc_fence_before();
        mbar_arrive(bar(P_READY + slot));
      }
      // ---- epilogue: O / l -> bf16 -> swizzled staging tile (the slot's Q buffer) -> TMA store
      if (ok && n_tiles > 0) ok = mbar_wait(bar(O_FULL), 0, abort_flag);
      if (ok) {
        tc_fence_after();
        const float inv = l > 0.f ? 1.f / l : 0.f;
        const uint32_t stage = q_smem + slot * kTileBytes;
#pragma unroll 1
        for (int c = 0; c < 4; ++c) {
          uint32_t o[32];
          if (n_tiles > 0) {
            tmem_ld32(o_t + c * 32, o);
            tmem_ld_wait();
          } else {
#pragma unroll
            for (int e = 0; e < 32; ++e) o[e] = 0u;
          }
#pragma unroll
          for (int jj = 0; jj < 4; ++jj) {
            uint32_t w[4];
#pragma unroll
            for (int e = 0; e < 4; ++e)
              w[e] = pack_bf16(__uint_as_float(o[jj * 8 + 2 * e]) * inv, __uint_as_float(o[jj * 8 + 2 * e + 1]) * inv);
            const int chunk = (c & 1) * 4 + jj;
            const uint32_t dst = stage + (uint32_t)(c >> 1) * kHalfBytes + (uint32_t)row_in_tile * 128u +
                                 (uint32_t)((chunk ^ (row_in_tile & 7)) << 4);
            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(w[0]), "r"(w[1]), "r"(w[2]), "r"(w[3])
                         : "memory");
          }
        }
        fence_proxy_async_smem();
        mbar_arrive(bar(O_STAGED + slot));                               // the four warps of this slot
        if (quarter == 0 && lane == 0 && mbar_wait(bar(O_STAGED + slot), 0, abort_flag)) {
          for (int h = 0; h < 2; ++h) tma_store_3d(&tmap_o, stage + h * kHalfBytes, h * 64, head0 + slot, q0);
          tma_store_commit();
          tma_store_wait<0>();
        }
        if (row < p.Tq)
          p.lse[(int64_t)(head0 + slot) * p.Tq + row] = l > 0.f ? (m_used + log2f(l)) * 0.6931471805599453f : -INFINITY;
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
  if (threadIdx.x == 0 && *abort_flag && p.status != nullptr) atomicOr(p.status, kStatusWaitTimedOut);
}

}  // namespace flash

// ----------------------------------------------------------------------------------------
// A [T, H, D] tensor whose last dimension is contiguous, seen as a 3-D map {D, H, T} and
// fetched in boxes of 64 head-dim elements x 1 head x `rows` tokens (128-byte swizzle).
static CUtensorMap make_tmap_thd(const at::Tensor& t, uint32_t rows) {
  TORCH_CHECK(t.dim() == 3 && t.stride(2) == 1, "flash: [T, H, D] tensor with contiguous last dimension expected");
  TORCH_CHECK((reinterpret_cast<uintptr_t>(t.data_ptr()) & 15) == 0, "flash: 16-byte aligned tensors expected");
  TORCH_CHECK((t.stride(0) * 2) % 16 == 0 && (t.stride(1) * 2) % 16 == 0, "flash: strides must be multiples of 16 bytes");
  CUtensorMap map;
  const cuuint64_t dims[3] = {(cuuint64_t)t.size(2), (cuuint64_t)t.size(1), (cuuint64_t)t.size(0)};
  const cuuint64_t strides[2] = {(cuuint64_t)t.stride(1) * 2, (cuuint64_t)t.stride(0) * 2};
  const cuuint32_t box[3] = {64, 1, rows};
  const cuuint32_t elem[3] = {1, 1, 1};
  const CUresult r = cuTensorMapEncodeTiled(&map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, t.data_ptr(), dims, strides, box,
                                            elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                            CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  TORCH_CHECK(r == CUDA_SUCCESS, "cuTensorMapEncodeTiled (flash) failed with code ", (int)r);
  return map;
}

static at::Tensor& flash_status_tensor(const at::Device& dev) {
  static std::vector<at::Tensor> per_device(64);
  auto& t = per_device[dev.index()];
  if (!t.defined()) t = at::zeros({1}, at::TensorOptions().dtype(at::kInt).device(dev));
  return t;
}

// q [Tq, Hq, 128], k / v [Tk, Hkv, 128] (bf16, last dimension contiguous) -> (o [Tq, Hq, 128], lse [Hq, Tq]).
// Query row i attends to keys kv_first[i] <= j <= i + causal_offset (causal) or all keys >= kv_first[i].
std::tuple<at::Tensor, at::Tensor> flash_fwd(const at::Tensor& q, const at::Tensor& k, const at::Tensor& v, double scale,
                                             bool causal, int64_t causal_offset,
                                             const c10::optional<at::Tensor>& kv_first) {
  using namespace flash;
  TORCH_CHECK(q.is_cuda() && k.is_cuda() && v.is_cuda());
  TORCH_CHECK(q.scalar_type() == at::kBFloat16 && k.scalar_type() == at::kBFloat16 && v.scalar_type() == at::kBFloat16);
  TORCH_CHECK(q.dim() == 3 && k.dim() == 3 && v.dim() == 3);
  TORCH_CHECK(q.size(2) == kD && k.size(2) == kD && v.size(2) == kD, "flash_fwd: head dimension must be 128");
  const int64_t Tq = q.size(0), Hq = q.size(1), Tk = k.size(0), Hkv = k.size(1);
  TORCH_CHECK(v.size(0) == Tk && v.size(1) == Hkv && Hq % Hkv == 0, "flash_fwd: inconsistent shapes");
  c10::cuda::CUDAGuard guard(q.device());
  C10_CUDA_CHECK(cudaSetDevice(q.device().index()));
  auto o = at::empty({Tq, Hq, kD}, q.options());
  auto lse = at::empty({Hq, Tq}, q.options().dtype(at::kFloat));
  if (Tq == 0) return {o, lse};
  TORCH_CHECK(Tk > 0, "flash_fwd: empty key sequence");
  const int group = (int)(Hq / Hkv);
  FwdParams p;
  p.Tq = (int)Tq; p.Tk = (int)Tk; p.Hq = (int)Hq; p.Hkv = (int)Hkv;
  p.causal = causal ? 1 : 0;
  p.causal_offset = (int)causal_offset;
  p.slots = group % 2 == 0 ? 2 : 1;
  p.ctas_per_kv_head = group / p.slots;
  p.scale_log2 = (float)(scale * 1.4426950408889634);
  p.kv_first = nullptr;
  if (kv_first.has_value() && kv_first->defined()) {
    TORCH_CHECK(kv_first->is_cuda() && kv_first->scalar_type() == at::kInt && kv_first->numel() == Tq &&
                kv_first->is_contiguous(), "flash_fwd: kv_first must be an int32 [Tq] CUDA tensor");
    p.kv_first = kv_first->data_ptr<int>();
  }
  p.lse = lse.data_ptr<float>();
  p.status = flash_status_tensor(q.device()).data_ptr<int>();
  const CUtensorMap tq = make_tmap_thd(q, kBM), tk = make_tmap_thd(k, kBN), tv = make_tmap_thd(v, kBN),
                    to = make_tmap_thd(o, kBM);
  constexpr uint32_t smem = 6 * kTileBytes + 1024 + 256;
  static bool attr_set = false;
  if (!attr_set) {
    C10_CUDA_CHECK(cudaFuncSetAttribute(flash_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    attr_set = true;
  }
  const int num_q_tiles = (int)((Tq + kBM - 1) / kBM);
  const int grid = num_q_tiles * (int)Hkv * p.ctas_per_kv_head;
  flash_fwd_kernel<<<grid, kThreadsFwd, smem, at::cuda::getCurrentCUDAStream()>>>(tq, tk, tv, to, p);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  return {o, lse};
}

int64_t flash_status(bool clear) {
  int dev = 0;
  cudaGetDevice(&dev);
  auto& t = flash_status_tensor(at::Device(at::kCUDA, dev));
  const int64_t v = t.item<int>();
  if (clear && v) t.zero_();
  return v;
}

}  // namespace tb200
