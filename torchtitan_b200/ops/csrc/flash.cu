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
#include <cstdlib>
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
  float* lse;              // [Hq, Tq] natural-log sum-exp of the scaled scores, row stride lse_stride
  int lse_stride;
  int debug;               // timing diagnostics: bit 0 skips the softmax math, bit 1 skips the MMAs (results are garbage)
  int* status;
  int window;              // > 0: query row i sees only keys j > i + causal_offset - window (sliding window; pipelined kernel only)
  const float* sinks;      // [Hq] per-head sink logit that joins the softmax denominator, or nullptr (pipelined kernel only)
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
      mbar_init(bar(P_READY + s), 4);      // one arrival per warp (lane 0 after __syncwarp)
      mbar_init(bar(O_STAGED + s), 4);
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
        if (p.debug & 2) return;
        const uint32_t qa = q_smem + slot * kTileBytes, ka = k_smem + st * kTileBytes;
#pragma unroll
        for (int k = 0; k < kD / 16; ++k) {
          const uint32_t off = (uint32_t)(k >> 2) * kHalfBytes + (uint32_t)(k & 3) * 32u;
          umma_bf16<1>(tmem_base + slot * 256, make_desc(qa + off, 16, 1024), make_desc(ka + off, 16, 1024), idesc_s,
                       k != 0 ? 1u : 0u);
        }
      };
      auto issue_pv = [&](int slot, int st, bool accumulate) {
        if (p.debug & 2) return;
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
        if (p.debug & 1) { tc_fence_before(); __syncwarp(); if (lane == 0) mbar_arrive(bar(P_READY + slot)); continue; }
        uint32_t r[4][32];
#pragma unroll
        for (int c = 0; c < 4; ++c) tmem_ld32(s_t + c * 32, r[c]);
        tmem_ld_wait();
        const int c0 = (j_lo + i) * kBN;
        const bool edge = (c0 + kBN - 1 > hi) || (c0 < lo);
        // Row maximum of the raw scores (the scale is positive, so it commutes with max): four
        // independent partial maxima keep the dependent chain at 32 instead of 128 instructions.
        if (edge) {
#pragma unroll
          for (int c = 0; c < 4; ++c)
#pragma unroll
            for (int e = 0; e < 32; ++e) {
              const int col = c0 + c * 32 + e;
              if (col > hi || col < lo) r[c][e] = __float_as_uint(-INFINITY);
            }
        }
        float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
        for (int c = 0; c < 4; ++c)
#pragma unroll
          for (int e = 0; e < 32; ++e) mx[e & 3] = fmaxf(mx[e & 3], __uint_as_float(r[c][e]));
        const float m_tile = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3])) * p.scale_log2;
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
        // P = exp2(S scale - m): one FFMA and one MUFU per element; four partial row sums
        const float neg_m = (m_used == -INFINITY) ? 0.f : -m_used;
        float ls[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint32_t pk[16];
#pragma unroll
          for (int e = 0; e < 16; ++e) {
            const float p0 = exp2f(fmaf(__uint_as_float(r[c][2 * e]), p.scale_log2, neg_m));
            const float p1 = exp2f(fmaf(__uint_as_float(r[c][2 * e + 1]), p.scale_log2, neg_m));
            ls[e & 3] += p0 + p1;
            pk[e] = pack_bf16(p0, p1);
          }
          tmem_st16(s_t + c * 16, pk);
        }
        l += (ls[0] + ls[1]) + (ls[2] + ls[3]);
        tmem_st_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar(P_READY + slot));
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
        __syncwarp();
        if (lane == 0) mbar_arrive(bar(O_STAGED + slot));                               // the four warps of this slot
        if (quarter == 0 && lane == 0 && mbar_wait(bar(O_STAGED + slot), 0, abort_flag)) {
          for (int h = 0; h < 2; ++h) tma_store_3d(&tmap_o, stage + h * kHalfBytes, h * 64, head0 + slot, q0);
          tma_store_commit();
          tma_store_wait<0>();
        }
        if (row < p.Tq)
          p.lse[(int64_t)(head0 + slot) * p.lse_stride + row] = l > 0.f ? (m_used + log2f(l)) * 0.6931471805599453f : -INFINITY;
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


// -----------------------------------------------------------------------------------------
// Forward, software-pipelined over half tiles (the default forward).
//
// Same roles, shared-memory and tensor-memory layout as flash_fwd_kernel, but each 128-key tile is
// processed as two halves of 64 keys, each with its own S accumulator (64 TMEM columns), its own
// packed P (the first 32 of those columns) and its own pair of barriers.  Per slot the chain
// S -> softmax -> P.V of one half overlaps with the other half's: while the slot's softmax warps
// work on half h, the tensor pipe runs P.V of half 1-h and the next tile's S for it, so the softmax
// warps (the exponentials) run back to back instead of waiting for the MMAs of their own slot.
//
// Rescaling O when the running maximum grows (rare: the threshold is 2^8) touches an accumulator
// that a P.V MMA of the other half may still be adding to.  The MMA warp follows every P.V with
// the next S of the same half and a commit on that half's S_FULL barrier (a bare commit after the
// last tile), so "S_FULL of the next work item is complete" implies "every P.V issued so far for
// this slot is complete"; a row that must rescale waits for that barrier first.
//
// kEmu of every 8 exponentials are evaluated on the FMA pipe (round-to-nearest range reduction,
// cubic polynomial, exponent patched in with an integer add; relative error 1e-4, below bf16
// rounding of P), which takes load off the 16-per-clock MUFU unit that otherwise bounds the loop.
// kPacked uses the two-wide fp32 instructions (fma.rn.f32x2 / add.f32x2) for the scale-and-shift
// and the row sums.
__device__ __forceinline__ uint64_t pack2(float lo, float hi) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ void unpack2(uint64_t v, float& lo, float& hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ uint64_t fma2(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}
__device__ __forceinline__ uint64_t add2(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("add.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ float max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}
__device__ __forceinline__ float ex2_mufu(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// 2^x for x in [-126, 127] on the FMA pipe.
__device__ __forceinline__ float ex2_poly(float x) {
  x = fmaxf(x, -126.f);
  const float fl = x + 12582912.f;                 // 1.5 * 2^23: the integer nearest to x sits in the low mantissa bits
  const float f = x - (fl - 12582912.f);           // in [-0.5, 0.5]
  float y = fmaf(f, 0.05500866f, 0.24221057f);
  y = fmaf(y, f, 0.69328291f);
  y = fmaf(y, f, 1.0f);
  return __uint_as_float(__float_as_uint(y) + (__float_as_uint(fl) << 23));
}

template <int kEmu, bool kPacked>
__global__ void __launch_bounds__(kThreadsFwd, 1)
flash_fwd_pipe_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                      const __grid_constant__ CUtensorMap tmap_v, const __grid_constant__ CUtensorMap tmap_o,
                      const FwdParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* gen_base = smem_raw + (base - raw);
  const uint32_t q_smem = base;
  const uint32_t k_smem = base + 2 * kTileBytes;
  const uint32_t v_smem = base + 4 * kTileBytes;
  const uint32_t bar_base = base + 6 * kTileBytes;
  // S_FULL / P_READY: index = slot * 2 + half
  enum { Q_FULL = 0, K_FULL = 1, K_EMPTY = 3, V_FULL = 5, V_EMPTY = 7, S_FULL = 9, P_READY = 13, O_FULL = 17, O_STAGED = 18,
         NBAR = 20 };
  auto bar = [&](int i) { return bar_base + 8u * i; };
  uint32_t* tmem_ptr_smem = reinterpret_cast<uint32_t*>(gen_base + 6 * kTileBytes + 8 * NBAR);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_ptr_smem + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  constexpr int kHN = kBN / 2;   // keys per half tile

  const int num_q_tiles = (p.Tq + kBM - 1) / kBM;
  const int per_tile = p.Hkv * p.ctas_per_kv_head;
  const int q_tile = num_q_tiles - 1 - (int)blockIdx.x / per_tile;
  const int rem = (int)blockIdx.x % per_tile;
  const int kv_head = rem / p.ctas_per_kv_head;
  const int group = p.Hq / p.Hkv;
  const int head0 = kv_head * group + (rem % p.ctas_per_kv_head) * p.slots;
  const int q0 = q_tile * kBM;
  const int num_k_tiles = (p.Tk + kBN - 1) / kBN;
  int j_hi = num_k_tiles - 1;
  if (p.causal) j_hi = min(j_hi, (min(q0 + kBM - 1, p.Tq - 1) + p.causal_offset) / kBN);
  int first_key = 0;                                                   // lowest key any row of this block sees
  if (p.kv_first != nullptr) first_key = max(0, p.kv_first[q0]);      // kv_first is non-decreasing
  if (p.window > 0) first_key = max(first_key, q0 + p.causal_offset - p.window + 1);
  const int j_lo = first_key / kBN;
  const int n_tiles = j_hi - j_lo + 1;                                 // may be <= 0: nothing visible
  const int n_items = 2 * n_tiles;

  if (threadIdx.x == 0) {
    mbar_init(bar(Q_FULL), 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(bar(K_FULL + s), 1);
      mbar_init(bar(K_EMPTY + s), 1);
      mbar_init(bar(V_FULL + s), 1);
      mbar_init(bar(V_EMPTY + s), 1);
      mbar_init(bar(O_STAGED + s), 4);
    }
    for (int s = 0; s < 4; ++s) {
      mbar_init(bar(S_FULL + s), 1);
      mbar_init(bar(P_READY + s), 4);      // one arrival per warp (lane 0 after __syncwarp)
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
      const uint32_t idesc_s = make_idesc(false, false, kBM, kHN);   // Q, K both K-major; 64 keys per instruction
      const uint32_t idesc_pv = make_idesc(false, true, kBM, kD);    // V is [keys, head dim]: MN-major B
      auto issue_s = [&](int slot, int half, int st) {
        if (p.debug & 2) return;
        const uint32_t qa = q_smem + slot * kTileBytes;
        const uint32_t ka = k_smem + st * kTileBytes + (uint32_t)half * (kHN * 128u);   // key rows [64 half, 64 half + 64)
#pragma unroll
        for (int k = 0; k < kD / 16; ++k) {
          const uint32_t off = (uint32_t)(k >> 2) * kHalfBytes + (uint32_t)(k & 3) * 32u;
          umma_bf16<1>(tmem_base + slot * 256 + half * kHN, make_desc(qa + off, 16, 1024), make_desc(ka + off, 16, 1024),
                       idesc_s, k != 0 ? 1u : 0u);
        }
      };
      auto issue_pv = [&](int slot, int half, int st, bool accumulate) {
        if (p.debug & 2) return;
        const uint32_t va = v_smem + st * kTileBytes + (uint32_t)half * (kHN / 16) * 2048u;
#pragma unroll
        for (int k = 0; k < kHN / 16; ++k)   // 16 keys per step: 8 packed columns of P, 16 rows (2048 B) of V
          umma_bf16_ts(tmem_base + slot * 256 + 128, tmem_base + slot * 256 + half * kHN + k * 8,
                       make_desc(va + k * 2048, kHalfBytes, 1024), idesc_pv, (accumulate || k != 0) ? 1u : 0u);
      };
      bool ok = mbar_wait(bar(Q_FULL), 0, abort_flag) && mbar_wait(bar(K_FULL), 0, abort_flag);
      if (ok) {
        tc_fence_after();
        for (int h = 0; h < 2; ++h)
          for (int s = 0; s < p.slots; ++s) {
            issue_s(s, h, 0);
            umma_commit(bar(S_FULL + s * 2 + h));
          }
        umma_commit(bar(K_EMPTY));
      }
      for (int w = 0; w < n_items && ok; ++w) {
        const int i = w >> 1, h = w & 1, st = i & 1;
        if (h == 0 && !mbar_wait(bar(V_FULL + st), (i >> 1) & 1u, abort_flag)) { ok = false; break; }
        for (int s = 0; s < p.slots && ok; ++s) {
          if (!mbar_wait(bar(P_READY + s * 2 + h), i & 1u, abort_flag)) { ok = false; break; }
          tc_fence_after();
          issue_pv(s, h, st, w > 0);
          if (h == 1 && s == p.slots - 1) umma_commit(bar(V_EMPTY + st));
          if (i + 1 < n_tiles) {
            const int st1 = (i + 1) & 1;
            if (s == 0 && h == 0 && !mbar_wait(bar(K_FULL + st1), ((i + 1) >> 1) & 1u, abort_flag)) { ok = false; break; }
            tc_fence_after();
            issue_s(s, h, st1);
            umma_commit(bar(S_FULL + s * 2 + h));
            if (h == 1 && s == p.slots - 1) umma_commit(bar(K_EMPTY + st1));
          } else {
            umma_commit(bar(S_FULL + s * 2 + h));   // no next S: the commit still tells a rescaling row that this P.V is done
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
      int lo = p.kv_first != nullptr ? p.kv_first[min(row, p.Tq - 1)] : 0;                // first visible key
      const int hi = min(p.Tk - 1, p.causal ? row + p.causal_offset : p.Tk - 1);           // last visible key
      if (p.window > 0) lo = max(lo, row + p.causal_offset - p.window + 1);
      float m_used = -INFINITY, l = 0.f;
      bool ok = true;
      for (int w = 0; w < n_items; ++w) {
        const int i = w >> 1, h = w & 1;
        if (!mbar_wait(bar(S_FULL + slot * 2 + h), i & 1u, abort_flag)) { ok = false; break; }
        tc_fence_after();
        if (p.debug & 1) { tc_fence_before(); __syncwarp(); if (lane == 0) mbar_arrive(bar(P_READY + slot * 2 + h)); continue; }
        uint32_t r[2][32];
        tmem_ld32(s_t + h * kHN, r[0]);
        tmem_ld32(s_t + h * kHN + 32, r[1]);
        tmem_ld_wait();
        const int c0 = (j_lo + i) * kBN + h * kHN;
        const bool edge = (c0 + kHN - 1 > hi) || (c0 < lo);
        if (edge) {
#pragma unroll
          for (int c = 0; c < 2; ++c)
#pragma unroll
            for (int e = 0; e < 32; ++e) {
              const int col = c0 + c * 32 + e;
              if (col > hi || col < lo) r[c][e] = __float_as_uint(-INFINITY);
            }
        }
        // row maximum of the raw scores: four independent chains of three-input maxima
        float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
        for (int c = 0; c < 2; ++c)
#pragma unroll
          for (int e = 0; e < 32; e += 2)
            mx[(e >> 1) & 3] = max3(mx[(e >> 1) & 3], __uint_as_float(r[c][e]), __uint_as_float(r[c][e + 1]));
        const float m_tile = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3])) * p.scale_log2;
        const float m_new = fmaxf(m_used, m_tile);
        if (__any_sync(0xffffffffu, m_new > m_used + kRescaleThreshold)) {
          // every row of this warp moves to its own new maximum; O and l are rescaled once all P.V MMAs issued
          // so far for this slot have completed (see the header comment)
          if (w > 0) {
            if (!mbar_wait(bar(S_FULL + slot * 2 + (1 - h)), ((w + 1) >> 1) & 1u, abort_flag)) { ok = false; break; }
            tc_fence_after();
          }
          const float alpha = (m_used == -INFINITY) ? 0.f : ex2_mufu(m_used - m_new);
          l *= alpha;
          if (w > 0) {
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
        // P = exp2(S scale - m)
        const float neg_m = (m_used == -INFINITY) ? 0.f : -m_used;
        float lsum;
        if constexpr (kPacked) {
          const uint64_t sc2 = pack2(p.scale_log2, p.scale_log2), nm2 = pack2(neg_m, neg_m);
          uint64_t ls2[2] = {pack2(0.f, 0.f), pack2(0.f, 0.f)};
#pragma unroll
          for (int c = 0; c < 2; ++c) {
            uint32_t pk[16];
#pragma unroll
            for (int e = 0; e < 16; ++e) {
              float x0, x1;
              unpack2(fma2(pack2(__uint_as_float(r[c][2 * e]), __uint_as_float(r[c][2 * e + 1])), sc2, nm2), x0, x1);
              float p0, p1;
              if (!edge && (e & 3) < kEmu / 2) {
                p0 = ex2_poly(x0);
                p1 = ex2_poly(x1);
              } else {
                p0 = ex2_mufu(x0);
                p1 = ex2_mufu(x1);
              }
              ls2[e & 1] = add2(ls2[e & 1], pack2(p0, p1));
              pk[e] = pack_bf16(p0, p1);
            }
            tmem_st16(s_t + h * kHN + c * 16, pk);
          }
          float a0, a1, b0, b1;
          unpack2(ls2[0], a0, a1);
          unpack2(ls2[1], b0, b1);
          lsum = (a0 + a1) + (b0 + b1);
        } else {
          float ls[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
          for (int c = 0; c < 2; ++c) {
            uint32_t pk[16];
#pragma unroll
            for (int e = 0; e < 16; ++e) {
              const float x0 = fmaf(__uint_as_float(r[c][2 * e]), p.scale_log2, neg_m);
              const float x1 = fmaf(__uint_as_float(r[c][2 * e + 1]), p.scale_log2, neg_m);
              float p0, p1;
              if (!edge && (e & 3) < kEmu / 2) {
                p0 = ex2_poly(x0);
                p1 = ex2_poly(x1);
              } else {
                p0 = ex2_mufu(x0);
                p1 = ex2_mufu(x1);
              }
              ls[e & 3] += p0 + p1;
              pk[e] = pack_bf16(p0, p1);
            }
            tmem_st16(s_t + h * kHN + c * 16, pk);
          }
          lsum = (ls[0] + ls[1]) + (ls[2] + ls[3]);
        }
        l += lsum;
        tmem_st_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar(P_READY + slot * 2 + h));
      }
      // ---- epilogue: O / l -> bf16 -> swizzled staging tile (the slot's Q buffer) -> TMA store
      if (ok && n_tiles > 0) ok = mbar_wait(bar(O_FULL), 0, abort_flag);
      if (ok) {
        tc_fence_after();
        // an attention sink adds exp(sink) to the denominator and nothing to the numerator
        float l_tot = l;
        const float sink2 = p.sinks != nullptr ? p.sinks[head0 + slot] * 1.4426950408889634f : -INFINITY;
        float m_fin = m_used;
        if (p.sinks != nullptr) {
          if (m_used == -INFINITY) { m_fin = sink2; l_tot = 1.f; }
          else l_tot = l + ex2_mufu(sink2 - m_used);
        }
        const float inv = (l > 0.f) ? 1.f / l_tot : 0.f;
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
            uint32_t wv[4];
#pragma unroll
            for (int e = 0; e < 4; ++e)
              wv[e] = pack_bf16(__uint_as_float(o[jj * 8 + 2 * e]) * inv, __uint_as_float(o[jj * 8 + 2 * e + 1]) * inv);
            const int chunk = (c & 1) * 4 + jj;
            const uint32_t dst = stage + (uint32_t)(c >> 1) * kHalfBytes + (uint32_t)row_in_tile * 128u +
                                 (uint32_t)((chunk ^ (row_in_tile & 7)) << 4);
            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(wv[0]), "r"(wv[1]), "r"(wv[2]), "r"(wv[3])
                         : "memory");
          }
        }
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar(O_STAGED + slot));                               // the four warps of this slot
        if (quarter == 0 && lane == 0 && mbar_wait(bar(O_STAGED + slot), 0, abort_flag)) {
          for (int h = 0; h < 2; ++h) tma_store_3d(&tmap_o, stage + h * kHalfBytes, h * 64, head0 + slot, q0);
          tma_store_commit();
          tma_store_wait<0>();
        }
        if (row < p.Tq)
          p.lse[(int64_t)(head0 + slot) * p.lse_stride + row] =
              l_tot > 0.f ? (m_fin + log2f(l_tot)) * 0.6931471805599453f : -INFINITY;
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


// =========================================================================================
// Backward, in two kernels that share no memory traffic besides their inputs, so that nothing
// is accumulated through global memory (an earlier single kernel that reduced dQ partials with
// TMA reduce-add into an fp32 buffer ran at 9 % tensor-pipe utilisation, bound by the L2
// reduction rate).
//
// flash_bwd_dkv_kernel.  One CTA owns a block of 128 keys of one key/value head and walks over
// every query head of its group and every block of 64 query rows that can see those keys.
// Scores are computed transposed (keys on the TMEM lanes), so the probabilities feed the dV and
// dK MMAs straight from tensor memory, and dK / dV accumulate in tensor memory over all query
// heads of the group and leave once.  Per step:
//     S^T  = K . Q^T,  dP^T = V . dO^T                      (tcgen05.mma, shared-memory operands)
//     P^T  = exp2(S^T c - lse),  dS^T = P^T (dP^T - delta) scale     (8 warps, one key row each,
//            written back over S^T / dP^T as packed bf16)
//     dV  += P^T . dO,  dK += dS^T . Q                      (A operand from tensor memory)
// S^T / dP^T are double buffered: the MMAs of step t+1 run while the warps work on step t.
//   warp 0       TMA producer (K, V once; Q and dO blocks through a four-stage ring)
//   warp 1       TMEM allocation, MMA issue
//   warps 2..17  lane quarter = warp % 4, column group (16 query columns) = (warp - 2) / 4
// Tensor memory: S^T [0,64) [64,128)   dP^T [128,192) [192,256)   dK [256,384)   dV [384,512)
constexpr int kBQ = 64;                       // query rows per step
constexpr int kMathGroups = 4;                // column groups: 4 warps (one per TMEM lane quarter) each
constexpr int kThreadsBwd = 64 + 128 * kMathGroups;
constexpr int kRing = 4;
constexpr uint32_t kQBytes = kBQ * kD * 2;    // 16 KB: 64 x 128 bf16 (two 64-column halves of 8 KB)

struct BwdParams {
  int Tq, Tk, Hq, Hkv;
  int causal, causal_offset;
  float scale, scale_log2;
  const int* kv_first;     // [Tq] or nullptr
  const float* lse;        // [Hq, Tq]: -lse log2(e) (pre-scaled by flash_delta_kernel), row stride `stat_stride`
  const float* delta;      // [Hq, Tq]: -rowsum(dO * O) scale, row stride `stat_stride`
  int debug;               // timing diagnostics: bit 0 skips the warps' math, bit 1 skips the MMAs (results are garbage)
  int stat_stride;         // a multiple of 64 floats, so that 64-row slices can be fetched with bulk copies
  int* status;
  int window;              // > 0: query row i sees only keys j > i + causal_offset - window
};

__global__ void __launch_bounds__(kThreadsBwd, 1)
flash_bwd_dkv_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_do,
                     const __grid_constant__ CUtensorMap tmap_k, const __grid_constant__ CUtensorMap tmap_v,
                     const __grid_constant__ CUtensorMap tmap_dk, const __grid_constant__ CUtensorMap tmap_dv,
                     const BwdParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* gen_base = smem_raw + (base - raw);
  // shared memory: K | V | ring[kRing] of (Q, dO) | barriers
  const uint32_t k_smem = base;
  const uint32_t v_smem = base + kTileBytes;
  const uint32_t ring_smem = base + 2 * kTileBytes;                 // stage s: Q at +s*32K, dO at +s*32K+16K
  constexpr uint32_t kStatOff = 2 * kTileBytes + kRing * 2 * kQBytes;   // per stage: lse[64] | delta[64] (fp32)
  const uint32_t stat_smem = base + kStatOff;
  constexpr uint32_t kBarOff = kStatOff + kRing * 512;
  const uint32_t bar_base = base + kBarOff;
  enum { KV_FULL = 0, R_FULL = 1, R_EMPTY = 1 + kRing, ST_FULL = 1 + 2 * kRing, PS_READY = 3 + 2 * kRing,
         ALL_DONE = 5 + 2 * kRing, OUT_STAGED = 6 + 2 * kRing, NBAR = 7 + 2 * kRing };
  auto bar = [&](int i) { return bar_base + 8u * i; };
  uint32_t* tmem_ptr_smem = reinterpret_cast<uint32_t*>(gen_base + kBarOff + 8 * NBAR);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_ptr_smem + 1);
  int* q_range = reinterpret_cast<int*>(tmem_ptr_smem + 2);   // [q_lo, n_sub]

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int num_k_tiles = (p.Tk + kBN - 1) / kBN;
  // causal: the first key blocks see the most query rows; they are scheduled first
  const int j = (int)blockIdx.x / p.Hkv;
  const int kv_head = (int)blockIdx.x % p.Hkv;
  const int group = p.Hq / p.Hkv;
  const int k0 = j * kBN;

  if (threadIdx.x == 0) {
    mbar_init(bar(KV_FULL), 1);
    for (int s = 0; s < kRing; ++s) {
      mbar_init(bar(R_FULL + s), 1);
      mbar_init(bar(R_EMPTY + s), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(bar(ST_FULL + b), 1);
      mbar_init(bar(PS_READY + b), 4 * kMathGroups);   // one arrival per warp
    }
    mbar_init(bar(ALL_DONE), 1);
    mbar_init(bar(OUT_STAGED), 4 * kMathGroups);
    *abort_flag = 0;
    mbar_fence_init();
    // query rows that can see this key block: [q_lo, q_hi)
    int q_lo = 0, q_hi = p.Tq;
    if (p.causal) q_lo = max(0, k0 - p.causal_offset);
    // sliding window: the last key of this block is visible up to query row last_key - offset + window - 1
    if (p.window > 0) q_hi = max(0, min(q_hi, min(k0 + kBN, p.Tk) - p.causal_offset + p.window - 1));
    if (p.kv_first != nullptr) {
      // kv_first is non-decreasing: rows from the first one whose first key lies beyond this block see nothing
      int a = 0, b = p.Tq;
      const int last_key = min(k0 + kBN, p.Tk) - 1;
      while (a < b) {
        const int mid = (a + b) >> 1;
        if (p.kv_first[mid] <= last_key) a = mid + 1; else b = mid;
      }
      q_hi = min(q_hi, a);
    }
    q_lo = (q_lo / kBQ) * kBQ;
    q_range[0] = q_lo;
    q_range[1] = q_hi > q_lo ? (q_hi - q_lo + kBQ - 1) / kBQ : 0;
    tma_prefetch_desc(&tmap_q);
    tma_prefetch_desc(&tmap_do);
    tma_prefetch_desc(&tmap_k);
    tma_prefetch_desc(&tmap_v);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_ptr_smem), 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_ptr_smem;
  const int q_lo = q_range[0];
  const int n_sub = q_range[1];
  const int n_iter = n_sub * group;
  constexpr uint32_t T_ST = 0, T_DPT = 128, T_DK = 256, T_DV = 384;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0 && n_iter > 0) {
      mbar_expect_tx(bar(KV_FULL), 2 * kTileBytes);
      for (int h = 0; h < 2; ++h) {
        tma_load_3d(k_smem + h * kHalfBytes, &tmap_k, bar(KV_FULL), h * 64, kv_head, k0);
        tma_load_3d(v_smem + h * kHalfBytes, &tmap_v, bar(KV_FULL), h * 64, kv_head, k0);
      }
      for (int t = 0; t < n_iter; ++t) {
        const int st = t % kRing;
        if (!mbar_wait(bar(R_EMPTY + st), ((t / kRing) & 1u) ^ 1u, abort_flag)) break;
        const int head = kv_head * group + t / n_sub;
        const int qs = q_lo + (t % n_sub) * kBQ;
        const uint32_t qa = ring_smem + st * 2 * kQBytes, doa = qa + kQBytes;
        mbar_expect_tx(bar(R_FULL + st), 2 * kQBytes + 512);
        for (int h = 0; h < 2; ++h) {
          tma_load_3d(qa + h * (kQBytes / 2), &tmap_q, bar(R_FULL + st), h * 64, head, qs);
          tma_load_3d(doa + h * (kQBytes / 2), &tmap_do, bar(R_FULL + st), h * 64, head, qs);
        }
        bulk_load(stat_smem + st * 512, p.lse + (int64_t)head * p.stat_stride + qs, 256, bar(R_FULL + st));
        bulk_load(stat_smem + st * 512 + 256, p.delta + (int64_t)head * p.stat_stride + qs, 256, bar(R_FULL + st));
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0 && n_iter > 0) {
      const uint32_t idesc_st = make_idesc(false, false, kBN, kBQ);   // K / V and Q / dO all K-major (head dim contiguous)
      const uint32_t idesc_acc = make_idesc(false, true, kBN, kD);    // A from TMEM, B = dO or Q as [query, head dim]: MN-major
      auto issue_scores = [&](int t) -> bool {
        const int st = t % kRing, b = t & 1;
        if (!mbar_wait(bar(R_FULL + st), (t / kRing) & 1u, abort_flag)) return false;
        tc_fence_after();
        if (p.debug & 2) { umma_commit(bar(ST_FULL + b)); return true; }
        const uint32_t qa = ring_smem + st * 2 * kQBytes, doa = qa + kQBytes;
#pragma unroll
        for (int k = 0; k < kD / 16; ++k) {
          // the two accumulators alternate, so consecutive MMAs do not depend on each other
          const uint32_t koff = (uint32_t)(k >> 2) * kHalfBytes + (uint32_t)(k & 3) * 32u;
          const uint32_t qoff = (uint32_t)(k >> 2) * (kQBytes / 2) + (uint32_t)(k & 3) * 32u;
          umma_bf16<1>(tmem_base + T_ST + b * 64, make_desc(k_smem + koff, 16, 1024), make_desc(qa + qoff, 16, 1024),
                       idesc_st, k != 0 ? 1u : 0u);
          umma_bf16<1>(tmem_base + T_DPT + b * 64, make_desc(v_smem + koff, 16, 1024), make_desc(doa + qoff, 16, 1024),
                       idesc_st, k != 0 ? 1u : 0u);
        }
        umma_commit(bar(ST_FULL + b));
        return true;
      };
      bool ok = mbar_wait(bar(KV_FULL), 0, abort_flag) && issue_scores(0);
      for (int t = 0; t < n_iter && ok; ++t) {
        const int st = t % kRing, b = t & 1;
        if (t + 1 < n_iter && !issue_scores(t + 1)) { ok = false; break; }
        if (!mbar_wait(bar(PS_READY + b), (t >> 1) & 1u, abort_flag)) { ok = false; break; }
        tc_fence_after();
        const uint32_t qa = ring_smem + st * 2 * kQBytes, doa = qa + kQBytes;
        if (!(p.debug & 2))
#pragma unroll
        for (int ks = 0; ks < kBQ / 16; ++ks) {   // 16 queries per step: 8 packed columns, 16 rows (2048 B) of dO / Q
          const uint32_t a_col = (uint32_t)b * 64u + (uint32_t)ks * 16u;
          umma_bf16_ts(tmem_base + T_DV, tmem_base + T_ST + a_col, make_desc(doa + ks * 2048, kQBytes / 2, 1024),
                       idesc_acc, (t > 0 || ks > 0) ? 1u : 0u);
          umma_bf16_ts(tmem_base + T_DK, tmem_base + T_DPT + a_col, make_desc(qa + ks * 2048, kQBytes / 2, 1024),
                       idesc_acc, (t > 0 || ks > 0) ? 1u : 0u);
        }
        umma_commit(bar(R_EMPTY + st));   // Q and dO of this stage are no longer read
      }
      if (ok) umma_commit(bar(ALL_DONE));
    }
  } else {
    // ------------------------------------------------------------------ softmax gradient, epilogue
    const int quarter = warp & 3;
    const int grp = (warp - 2) >> 2;               // 16 of the 64 query columns of a step
    const int r = quarter * 32 + lane;             // key row of this thread
    const int kv_idx = k0 + r;
    const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
    bool ok = true;
    const uint64_t sc2 = pack2(p.scale_log2, p.scale_log2), scl2 = pack2(p.scale, p.scale);
    int sub = 0, st = 0;                           // t % n_sub and t % kRing, kept without divisions
    uint32_t ring_par = 0;                         // (t / kRing) & 1
    for (int t = 0; t < n_iter; ++t) {
      const int b = t & 1;
      const int qc0 = q_lo + sub * kBQ + grp * 16;    // first query column of this thread
      if (!mbar_wait(bar(ST_FULL + b), (t >> 1) & 1u, abort_flag)) { ok = false; break; }
      tc_fence_after();
      if (p.debug & 1) {
        tc_fence_before(); __syncwarp(); if (lane == 0) mbar_arrive(bar(PS_READY + b));
        if (++sub == n_sub) sub = 0;
        if (++st == kRing) { st = 0; ring_par ^= 1u; }
        continue;
      }
      uint32_t sv[16], dv[16];
      tmem_ld16(tmem_base + lane_addr + T_ST + b * 64 + grp * 16, sv);
      tmem_ld16(tmem_base + lane_addr + T_DPT + b * 64 + grp * 16, dv);
      tmem_ld_wait();
      // -lse log2(e) and -delta scale of the 64 query rows of this step were staged next to Q / dO by the
      // producer (the stage's barrier has completed long ago: the MMAs that filled S^T waited on it)
      if (!mbar_wait(bar(R_FULL + st), ring_par, abort_flag)) { ok = false; break; }
      const uint32_t stat = stat_smem + (uint32_t)st * 512u + (uint32_t)grp * 64u;
      const bool edge = p.kv_first != nullptr || qc0 + 16 > p.Tq || k0 + kBN > p.Tk ||
                        (p.causal && qc0 + p.causal_offset < k0 + kBN - 1) ||
                        (p.window > 0 && qc0 + 15 + p.causal_offset - p.window + 1 > k0);
      uint32_t pk[8], dk[8];
#pragma unroll
      for (int g = 0; g < 4; ++g) {
        // two packed pairs of each statistic, ready to be the addend of a two-wide FMA
        uint64_t nl[2], nd[2];
        asm volatile("ld.shared.v2.b64 {%0, %1}, [%2];" : "=l"(nl[0]), "=l"(nl[1]) : "r"(stat + g * 16));
        asm volatile("ld.shared.v2.b64 {%0, %1}, [%2];" : "=l"(nd[0]), "=l"(nd[1]) : "r"(stat + 256 + g * 16));
#pragma unroll
        for (int h2 = 0; h2 < 2; ++h2) {
          const int i = g * 4 + h2 * 2;
          float x0, x1, d0, d1;
          unpack2(fma2(pack2(__uint_as_float(sv[i]), __uint_as_float(sv[i + 1])), sc2, nl[h2]), x0, x1);
          unpack2(fma2(pack2(__uint_as_float(dv[i]), __uint_as_float(dv[i + 1])), scl2, nd[h2]), d0, d1);
          float p0 = ex2_mufu(x0), p1 = ex2_mufu(x1);
          if (edge) {
#pragma unroll
            for (int u = 0; u < 2; ++u) {
              const int qi = qc0 + i + u;
              bool vis = qi < p.Tq && kv_idx < p.Tk;
              if (p.causal) vis = vis && kv_idx <= qi + p.causal_offset;
              if (p.window > 0) vis = vis && kv_idx > qi + p.causal_offset - p.window;
              if (p.kv_first != nullptr) vis = vis && kv_idx >= p.kv_first[min(qi, p.Tq - 1)];
              if (!vis) { if (u == 0) p0 = 0.f; else p1 = 0.f; }
            }
          }
          pk[2 * g + h2] = pack_bf16(p0, p1);
          dk[2 * g + h2] = pack_bf16(p0 * d0, p1 * d1);
        }
      }
      // packed P^T / dS^T of this group's 16 columns go to the first 8 of its own 16 TMEM columns
      tmem_st8(tmem_base + lane_addr + T_ST + b * 64 + grp * 16, pk);
      tmem_st8(tmem_base + lane_addr + T_DPT + b * 64 + grp * 16, dk);
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(PS_READY + b));
      if (++sub == n_sub) sub = 0;
      if (++st == kRing) { st = 0; ring_par ^= 1u; }
    }
    if (ok && n_iter > 0) ok = mbar_wait(bar(ALL_DONE), 0, abort_flag);
    // ---- dK, dV: tensor memory -> bf16 -> swizzled staging tiles (the Q / dO ring) -> TMA store
    if (ok) {
      tc_fence_after();
#pragma unroll 1
      for (int which = 0; which < 2; ++which) {
        // this thread's 32 head-dim columns: 64-column half grp / 2, 16-byte chunks (grp % 2) * 4 ...
        const uint32_t stage = ring_smem + which * kTileBytes + (grp >> 1) * kHalfBytes;
        uint32_t o[32];
        if (n_iter > 0) {
          tmem_ld32(tmem_base + lane_addr + (which ? T_DV : T_DK) + grp * 32, o);
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
            w[e] = pack_bf16(__uint_as_float(o[jj * 8 + 2 * e]), __uint_as_float(o[jj * 8 + 2 * e + 1]));
          const int chunk = (grp & 1) * 4 + jj;
          const uint32_t dst = stage + (uint32_t)r * 128u + (uint32_t)((chunk ^ (r & 7)) << 4);
          asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(w[0]), "r"(w[1]), "r"(w[2]), "r"(w[3])
                       : "memory");
        }
      }
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(OUT_STAGED));
      if (warp == 2 && lane == 0 && mbar_wait(bar(OUT_STAGED), 0, abort_flag)) {
        for (int h = 0; h < 2; ++h) {
          tma_store_3d(&tmap_dk, ring_smem + h * kHalfBytes, h * 64, kv_head, k0);
          tma_store_3d(&tmap_dv, ring_smem + kTileBytes + h * kHalfBytes, h * 64, kv_head, k0);
        }
        tma_store_commit();
        tma_store_wait<0>();
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

// flash_bwd_dq_kernel.  One CTA owns 128 query rows of one head and walks over the key blocks
// those rows can see (the forward's loop).  Per key block:
//     S = Q . K^T,  dP = dO . V^T             (tcgen05.mma, shared-memory operands)
//     dS = exp2(S c - lse) (dP - delta) scale  (16 warps: one query row, 32 keys per thread),
//          written as packed bf16 into its own tensor-memory columns
//     dQ += dS . K                             (A operand from tensor memory)
// The warps read S and dP of block i into registers and release both accumulators at once
// (SDP_FREE); the S and dP MMAs of block i+1 then run while the warps do the math of block i, so
// the exponentials run back to back and the tensor pipe stays fed.  dS has one buffer: the dQ MMA
// of block i is followed by a commit on DQ_DONE, which the warps wait for before they store dS of
// block i+1 (by then it has long completed).
//   warp 0 TMA producer (Q, dO once; K and V through two-stage rings), warp 1 MMA, warps 2..17 math
//   (lane quarter = warp % 4, group of 32 keys = (warp - 2) / 4)
// Tensor memory: S [0,128)   dP [128,256)   dS (packed bf16) [256,320)   dQ [384,512)
__global__ void __launch_bounds__(kThreadsBwd, 1)
flash_bwd_dq_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_do,
                    const __grid_constant__ CUtensorMap tmap_k, const __grid_constant__ CUtensorMap tmap_v,
                    const __grid_constant__ CUtensorMap tmap_dq, const BwdParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* gen_base = smem_raw + (base - raw);
  // shared memory: Q | dO | K ring[2] | V ring[2] | barriers
  const uint32_t q_smem = base;
  const uint32_t do_smem = base + kTileBytes;
  const uint32_t k_smem = base + 2 * kTileBytes;
  const uint32_t v_smem = base + 4 * kTileBytes;
  constexpr uint32_t kBarOff = 6 * kTileBytes;
  const uint32_t bar_base = base + kBarOff;
  enum { Q_FULL = 0, K_FULL = 1, K_EMPTY = 3, V_FULL = 5, V_EMPTY = 7, S_FULL = 9, DP_FULL = 10, DS_READY = 11, DQ_FULL = 12,
         OUT_STAGED = 13, SDP_FREE = 14, DQ_DONE = 15, NBAR = 16 };
  auto bar = [&](int i) { return bar_base + 8u * i; };
  uint32_t* tmem_ptr_smem = reinterpret_cast<uint32_t*>(gen_base + kBarOff + 8 * NBAR);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_ptr_smem + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int num_q_tiles = (p.Tq + kBM - 1) / kBM;
  const int q_tile = num_q_tiles - 1 - (int)blockIdx.x / p.Hq;      // longest rows first
  const int head = (int)blockIdx.x % p.Hq;
  const int kv_head = head / (p.Hq / p.Hkv);
  const int q0 = q_tile * kBM;
  const int num_k_tiles = (p.Tk + kBN - 1) / kBN;
  int j_hi = num_k_tiles - 1;
  if (p.causal) j_hi = min(j_hi, (min(q0 + kBM - 1, p.Tq - 1) + p.causal_offset) / kBN);
  int first_key = 0;
  if (p.kv_first != nullptr) first_key = max(0, p.kv_first[q0]);
  if (p.window > 0) first_key = max(first_key, q0 + p.causal_offset - p.window + 1);
  const int j_lo = first_key / kBN;
  const int n_tiles = j_hi - j_lo + 1;

  if (threadIdx.x == 0) {
    mbar_init(bar(Q_FULL), 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(bar(K_FULL + s), 1);
      mbar_init(bar(K_EMPTY + s), 1);
      mbar_init(bar(V_FULL + s), 1);
      mbar_init(bar(V_EMPTY + s), 1);
    }
    mbar_init(bar(S_FULL), 1);
    mbar_init(bar(DP_FULL), 1);
    mbar_init(bar(SDP_FREE), 4 * kMathGroups);
    mbar_init(bar(DQ_DONE), 1);
    mbar_init(bar(DS_READY), 4 * kMathGroups);
    mbar_init(bar(DQ_FULL), 1);
    mbar_init(bar(OUT_STAGED), 4 * kMathGroups);
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmap_q);
    tma_prefetch_desc(&tmap_do);
    tma_prefetch_desc(&tmap_k);
    tma_prefetch_desc(&tmap_v);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_ptr_smem), 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_ptr_smem;
  constexpr uint32_t T_S = 0, T_DP = 128, T_DS = 256, T_DQ = 384;

  if (warp == 0) {
    if (lane == 0 && n_tiles > 0) {
      mbar_expect_tx(bar(Q_FULL), 2 * kTileBytes);
      for (int h = 0; h < 2; ++h) {
        tma_load_3d(q_smem + h * kHalfBytes, &tmap_q, bar(Q_FULL), h * 64, head, q0);
        tma_load_3d(do_smem + h * kHalfBytes, &tmap_do, bar(Q_FULL), h * 64, head, q0);
      }
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
    if (lane == 0 && n_tiles > 0) {
      const uint32_t idesc_s = make_idesc(false, false, kBM, kBN);
      const uint32_t idesc_dq = make_idesc(false, true, kBM, kD);     // A = dS from TMEM, B = K as [key, head dim]
      // S and dP of one block: the two accumulators alternate, so that consecutive MMAs do not depend on each other
      auto issue_scores = [&](uint32_t k_tile, uint32_t v_tile) {
        if (p.debug & 2) return;
#pragma unroll
        for (int k = 0; k < kD / 16; ++k) {
          const uint32_t off = (uint32_t)(k >> 2) * kHalfBytes + (uint32_t)(k & 3) * 32u;
          umma_bf16<1>(tmem_base + T_S, make_desc(q_smem + off, 16, 1024), make_desc(k_tile + off, 16, 1024), idesc_s,
                       k != 0 ? 1u : 0u);
          umma_bf16<1>(tmem_base + T_DP, make_desc(do_smem + off, 16, 1024), make_desc(v_tile + off, 16, 1024), idesc_s,
                       k != 0 ? 1u : 0u);
        }
      };
      bool ok = mbar_wait(bar(Q_FULL), 0, abort_flag) && mbar_wait(bar(K_FULL), 0, abort_flag) &&
                mbar_wait(bar(V_FULL), 0, abort_flag);
      if (ok) {
        tc_fence_after();
        issue_scores(k_smem, v_smem);
        umma_commit(bar(S_FULL));
        umma_commit(bar(DP_FULL));
        umma_commit(bar(V_EMPTY));
      }
      for (int i = 0; i < n_tiles && ok; ++i) {
        const int st = i & 1;
        if (i + 1 < n_tiles) {
          const int s1 = (i + 1) & 1;
          // the warps hold S and dP of block i in registers: both accumulators take the next block now
          if (!mbar_wait(bar(SDP_FREE), i & 1u, abort_flag)) { ok = false; break; }
          if (!mbar_wait(bar(K_FULL + s1), ((i + 1) >> 1) & 1u, abort_flag)) { ok = false; break; }
          if (!mbar_wait(bar(V_FULL + s1), ((i + 1) >> 1) & 1u, abort_flag)) { ok = false; break; }
          tc_fence_after();
          issue_scores(k_smem + s1 * kTileBytes, v_smem + s1 * kTileBytes);
          umma_commit(bar(S_FULL));
          umma_commit(bar(DP_FULL));
          umma_commit(bar(V_EMPTY + s1));
        }
        if (!mbar_wait(bar(DS_READY), i & 1u, abort_flag)) { ok = false; break; }
        tc_fence_after();
        if (!(p.debug & 2))
#pragma unroll
        for (int ks = 0; ks < kBN / 16; ++ks)   // 16 keys per step: 8 packed columns of dS, 16 rows (2048 B) of K
          umma_bf16_ts(tmem_base + T_DQ, tmem_base + T_DS + (uint32_t)ks * 8u,
                       make_desc(k_smem + st * kTileBytes + ks * 2048, kHalfBytes, 1024), idesc_dq,
                       (i > 0 || ks > 0) ? 1u : 0u);
        umma_commit(bar(K_EMPTY + st));
        umma_commit(bar(DQ_DONE));
      }
      if (ok) umma_commit(bar(DQ_FULL));
    }
  } else {
    const int quarter = warp & 3;
    const int grp = (warp - 2) >> 2;               // 32 of the 128 keys of a block
    const int row_in_tile = quarter * 32 + lane;
    const int row = q0 + row_in_tile;
    const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
    const bool row_ok = row < p.Tq;
    const float l2 = row_ok ? -p.lse[(int64_t)head * p.stat_stride + row] : INFINITY;   // lse log2(e)
    const float dl = row_ok ? -p.delta[(int64_t)head * p.stat_stride + row] : 0.f;       // delta scale
    int lo = p.kv_first != nullptr ? p.kv_first[min(row, p.Tq - 1)] : 0;
    if (p.window > 0) lo = max(lo, row + p.causal_offset - p.window + 1);
    const int hi = min(p.Tk - 1, p.causal ? row + p.causal_offset : p.Tk - 1);
    bool ok = true;
    const uint64_t sc2 = pack2(p.scale_log2, p.scale_log2), nl2 = pack2(-l2, -l2);
    const uint64_t scl2 = pack2(p.scale, p.scale), ndl2 = pack2(-dl, -dl);
    for (int i = 0; i < n_tiles; ++i) {
      if (!mbar_wait(bar(S_FULL), i & 1u, abort_flag) || !mbar_wait(bar(DP_FULL), i & 1u, abort_flag)) {
        ok = false;
        break;
      }
      tc_fence_after();
      if (p.debug & 1) {
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar(SDP_FREE));
        if (i > 0 && !mbar_wait(bar(DQ_DONE), (i - 1) & 1u, abort_flag)) { ok = false; break; }
        if (lane == 0) mbar_arrive(bar(DS_READY));
        continue;
      }
      const int c0 = (j_lo + i) * kBN + grp * 32;
      const bool edge = (c0 + 31 > hi) || (c0 < lo);
      uint32_t sv[32], dv[32], out[16];
      tmem_ld32(tmem_base + lane_addr + T_S + grp * 32, sv);
      tmem_ld32(tmem_base + lane_addr + T_DP + grp * 32, dv);
      tmem_ld_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(SDP_FREE));
      if (edge) {
#pragma unroll
        for (int e = 0; e < 16; ++e) {
          float ds2[2];
#pragma unroll
          for (int u = 0; u < 2; ++u) {
            const int idx = 2 * e + u;
            const int col = c0 + idx;
            float pe = ex2_mufu(fmaf(__uint_as_float(sv[idx]), p.scale_log2, -l2));
            if (col > hi || col < lo) pe = 0.f;
            ds2[u] = pe * fmaf(__uint_as_float(dv[idx]), p.scale, -dl);
          }
          out[e] = pack_bf16(ds2[0], ds2[1]);
        }
      } else {
#pragma unroll
        for (int e = 0; e < 16; ++e) {
          float x0, x1, d0, d1;
          unpack2(fma2(pack2(__uint_as_float(sv[2 * e]), __uint_as_float(sv[2 * e + 1])), sc2, nl2), x0, x1);
          unpack2(fma2(pack2(__uint_as_float(dv[2 * e]), __uint_as_float(dv[2 * e + 1])), scl2, ndl2), d0, d1);
          out[e] = pack_bf16(ex2_mufu(x0) * d0, ex2_mufu(x1) * d1);
        }
      }
      // dS has a single buffer: the dQ MMA of the previous block must have read it
      if (i > 0) {
        if (!mbar_wait(bar(DQ_DONE), (i - 1) & 1u, abort_flag)) { ok = false; break; }
        tc_fence_after();
      }
      tmem_st16(tmem_base + lane_addr + T_DS + grp * 16, out);
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(DS_READY));
    }
    if (ok && n_tiles > 0) ok = mbar_wait(bar(DQ_FULL), 0, abort_flag);
    if (ok) {
      tc_fence_after();
      // dQ -> bf16 -> swizzled staging (the Q tile) -> TMA store; thread = (row, 32 head-dim columns)
      const uint32_t stage = q_smem + (grp >> 1) * kHalfBytes;
      uint32_t o[32];
      if (n_tiles > 0) {
        tmem_ld32(tmem_base + lane_addr + T_DQ + grp * 32, o);
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
          w[e] = pack_bf16(__uint_as_float(o[jj * 8 + 2 * e]), __uint_as_float(o[jj * 8 + 2 * e + 1]));
        const int chunk = (grp & 1) * 4 + jj;
        const uint32_t dst = stage + (uint32_t)row_in_tile * 128u + (uint32_t)((chunk ^ (row_in_tile & 7)) << 4);
        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(w[0]), "r"(w[1]), "r"(w[2]), "r"(w[3])
                     : "memory");
      }
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(OUT_STAGED));
      if (warp == 2 && lane == 0 && mbar_wait(bar(OUT_STAGED), 0, abort_flag)) {
        for (int h = 0; h < 2; ++h) tma_store_3d(&tmap_dq, q_smem + h * kHalfBytes, h * 64, head, q0);
        tma_store_commit();
        tma_store_wait<0>();
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

// The per-row statistics of the backward kernels, already in the form their inner loops add:
//   ndelta[h, t] = -scale sum_d dO[t, h, d] O[t, h, d]      nlse2[h, t] = -lse[h, t] log2(e)
// One warp per (token, head).
__global__ void flash_delta_kernel(const __nv_bfloat16* __restrict__ o, const __nv_bfloat16* __restrict__ d_o,
                                   const float* __restrict__ lse, int lse_stride, float* __restrict__ ndelta,
                                   float* __restrict__ nlse2, int T, int H, int stride, float scale) {
  const int64_t w = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (w >= (int64_t)T * H) return;
  const int t = (int)(w / H), h = (int)(w % H);
  const uint2 a = *reinterpret_cast<const uint2*>(o + w * kD + lane * 4);
  const uint2 b = *reinterpret_cast<const uint2*>(d_o + w * kD + lane * 4);
  const float2 a0 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&a.x));
  const float2 a1 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&a.y));
  const float2 b0 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&b.x));
  const float2 b1 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&b.y));
  const float s = warp_sum(a0.x * b0.x + a0.y * b0.y + a1.x * b1.x + a1.y * b1.y);
  if (lane == 0) {
    ndelta[(int64_t)h * stride + t] = -s * scale;
    nlse2[(int64_t)h * stride + t] = -lse[(int64_t)h * lse_stride + t] * 1.4426950408889634f;
  }
}

// Online-softmax merge of one block's normalised attention output into a running fp32 pair:
//   lse' = log(exp(lse_a) + exp(lse_b));  o' = o_a exp(lse_a - lse') + o_b exp(lse_b - lse').
// One warp per (token, head), four head-dim elements per lane; -inf (no visible key) contributes nothing.
__global__ void attn_merge_kernel(float* __restrict__ acc_o, float* __restrict__ acc_lse, const __nv_bfloat16* __restrict__ o,
                                  const float* __restrict__ lse, int T, int H, int acc_lse_stride, int lse_stride) {
  const int64_t w = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (w >= (int64_t)T * H) return;
  const int t = (int)(w / H), h = (int)(w % H);
  const float la = acc_lse[(int64_t)h * acc_lse_stride + t];
  const float lb = lse[(int64_t)h * lse_stride + t];
  const float mx = fmaxf(la, lb);
  float wa = 0.f, wb = 0.f, ln = -INFINITY;
  if (mx > -INFINITY) {
    const float ea = __expf(la - mx), eb = __expf(lb - mx);   // exp(-inf) = 0
    ln = mx + __logf(ea + eb);
    wa = ea / (ea + eb);
    wb = eb / (ea + eb);
  }
  float4 a = *reinterpret_cast<const float4*>(acc_o + w * kD + lane * 4);
  const uint2 b = *reinterpret_cast<const uint2*>(o + w * kD + lane * 4);
  const float2 b0 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&b.x));
  const float2 b1 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&b.y));
  a.x = a.x * wa + b0.x * wb;
  a.y = a.y * wa + b0.y * wb;
  a.z = a.z * wa + b1.x * wb;
  a.w = a.w * wa + b1.y * wb;
  *reinterpret_cast<float4*>(acc_o + w * kD + lane * 4) = a;
  __syncwarp();
  if (lane == 0) acc_lse[(int64_t)h * acc_lse_stride + t] = ln;
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

static int g_flash_debug = 0;
// Timing diagnostics that make the kernel skip part of its work (results are garbage by design).
// Refused unless the process was started with TB200_KERNEL_TIMING_DEBUG=1, so that no training
// job can switch them on by accident.
void flash_set_debug(int64_t v) {
  TORCH_CHECK(v == 0 || std::getenv("TB200_KERNEL_TIMING_DEBUG") != nullptr,
              "flash_set_debug: set TB200_KERNEL_TIMING_DEBUG=1 in the environment to enable the timing switches");
  g_flash_debug = (int)v;
}

static at::Tensor& flash_status_tensor(const at::Device& dev) {
  static std::vector<at::Tensor> per_device(64);
  auto& t = per_device[dev.index()];
  if (!t.defined()) t = at::zeros({1}, at::TensorOptions().dtype(at::kInt).device(dev));
  return t;
}

// Forward kernel selection: 0 = one 128-key tile per step (flash_fwd_kernel); 1..4 = the half-tile
// pipelined kernel with <kEmu, kPacked> = <0,false>, <0,true>, <2,true>, <4,true>.
static int g_flash_fwd_variant = -1;
void flash_set_fwd_variant(int64_t v) {
  TORCH_CHECK(v >= 0 && v <= 4, "flash_set_fwd_variant: 0..4");
  g_flash_fwd_variant = (int)v;
}
static int flash_fwd_variant() {
  if (g_flash_fwd_variant < 0) {
    const char* e = std::getenv("TB200_FLASH_FWD");
    g_flash_fwd_variant = (e != nullptr && e[0] >= '0' && e[0] <= '4' && e[1] == 0) ? e[0] - '0' : 0;
  }
  return g_flash_fwd_variant;
}

// q [Tq, Hq, 128], k / v [Tk, Hkv, 128] (bf16, last dimension contiguous) -> (o [Tq, Hq, 128], lse [Hq, Tq]).
// Query row i attends to keys max(kv_first[i], i + causal_offset - window + 1) <= j <= i + causal_offset
// (causal; window 0 = unlimited) or to all keys >= kv_first[i].  `sinks` [Hq] fp32: one extra logit per head
// that joins the softmax denominator only (its share of the probability mass is dropped); lse includes it.
std::tuple<at::Tensor, at::Tensor> flash_fwd(const at::Tensor& q, const at::Tensor& k, const at::Tensor& v, double scale,
                                             bool causal, int64_t causal_offset,
                                             const c10::optional<at::Tensor>& kv_first, int64_t window,
                                             const c10::optional<at::Tensor>& sinks) {
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
  // rows padded to a multiple of 64 floats: the backward fetches 64-row slices with bulk copies
  const int64_t Tpad = (Tq + 63) / 64 * 64;
  auto lse = at::empty({Hq, Tpad}, q.options().dtype(at::kFloat)).narrow(1, 0, Tq);
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
  p.lse_stride = (int)Tpad;
  p.debug = g_flash_debug;
  p.status = flash_status_tensor(q.device()).data_ptr<int>();
  p.window = 0;
  p.sinks = nullptr;
  TORCH_CHECK(window >= 0, "flash_fwd: window must be >= 0");
  int variant = flash_fwd_variant();
  if (window > 0) {
    TORCH_CHECK(causal, "flash_fwd: a sliding window needs causal attention");
    p.window = (int)window;
  }
  if (sinks.has_value() && sinks->defined()) {
    TORCH_CHECK(sinks->is_cuda() && sinks->scalar_type() == at::kFloat && sinks->numel() == Hq && sinks->is_contiguous(),
                "flash_fwd: sinks must be a float32 [Hq] CUDA tensor");
    p.sinks = sinks->data_ptr<float>();
  }
  if ((p.window > 0 || p.sinks != nullptr) && variant == 0) variant = 2;   // only the pipelined kernel has them
  const CUtensorMap tq = make_tmap_thd(q, kBM), tk = make_tmap_thd(k, kBN), tv = make_tmap_thd(v, kBN),
                    to = make_tmap_thd(o, kBM);
  constexpr uint32_t smem = 6 * kTileBytes + 1024 + 256;
  static bool attr_set = false;
  if (!attr_set) {
    C10_CUDA_CHECK(cudaFuncSetAttribute(flash_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    C10_CUDA_CHECK(cudaFuncSetAttribute(flash_fwd_pipe_kernel<0, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    C10_CUDA_CHECK(cudaFuncSetAttribute(flash_fwd_pipe_kernel<0, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    C10_CUDA_CHECK(cudaFuncSetAttribute(flash_fwd_pipe_kernel<2, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    C10_CUDA_CHECK(cudaFuncSetAttribute(flash_fwd_pipe_kernel<4, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    attr_set = true;
  }
  const int num_q_tiles = (int)((Tq + kBM - 1) / kBM);
  const int grid = num_q_tiles * (int)Hkv * p.ctas_per_kv_head;
  auto stream = at::cuda::getCurrentCUDAStream();
  switch (variant) {
    case 0: flash_fwd_kernel<<<grid, kThreadsFwd, smem, stream>>>(tq, tk, tv, to, p); break;
    case 1: flash_fwd_pipe_kernel<0, false><<<grid, kThreadsFwd, smem, stream>>>(tq, tk, tv, to, p); break;
    case 2: flash_fwd_pipe_kernel<0, true><<<grid, kThreadsFwd, smem, stream>>>(tq, tk, tv, to, p); break;
    case 4: flash_fwd_pipe_kernel<4, true><<<grid, kThreadsFwd, smem, stream>>>(tq, tk, tv, to, p); break;
    default: flash_fwd_pipe_kernel<2, true><<<grid, kThreadsFwd, smem, stream>>>(tq, tk, tv, to, p); break;
  }
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  return {o, lse};
}

// (dO [Tq, Hq, 128] contiguous, q, k, v, o, lse from the forward) -> (dq, dk, dv).  The three
// outputs may be given as views (last dimension contiguous), e.g. slices of one packed gradient.
// With attention sinks nothing changes here: lse from the forward already contains the sink, so
// exp(s - lse) are the probabilities of the real keys; the caller derives the sink's own gradient
// from lse and delta.
std::tuple<at::Tensor, at::Tensor, at::Tensor> flash_bwd(const at::Tensor& d_o, const at::Tensor& q, const at::Tensor& k,
                                                         const at::Tensor& v, const at::Tensor& o, const at::Tensor& lse,
                                                         double scale, bool causal, int64_t causal_offset,
                                                         const c10::optional<at::Tensor>& kv_first,
                                                         const c10::optional<at::Tensor>& dq_out,
                                                         const c10::optional<at::Tensor>& dk_out,
                                                         const c10::optional<at::Tensor>& dv_out, int64_t window) {
  using namespace flash;
  TORCH_CHECK(d_o.is_cuda() && q.is_cuda() && k.is_cuda() && v.is_cuda() && o.is_cuda() && lse.is_cuda());
  TORCH_CHECK(d_o.scalar_type() == at::kBFloat16 && q.scalar_type() == at::kBFloat16 && k.scalar_type() == at::kBFloat16 &&
              v.scalar_type() == at::kBFloat16 && o.scalar_type() == at::kBFloat16 && lse.scalar_type() == at::kFloat);
  const int64_t Tq = q.size(0), Hq = q.size(1), Tk = k.size(0), Hkv = k.size(1);
  TORCH_CHECK(q.size(2) == kD && k.size(2) == kD && v.size(2) == kD, "flash_bwd: head dimension must be 128");
  TORCH_CHECK(o.is_contiguous() && d_o.is_contiguous(), "flash_bwd: o and dO must be contiguous");
  TORCH_CHECK(o.size(0) == Tq && o.size(1) == Hq && d_o.sizes() == o.sizes() && lse.size(0) == Hq && lse.size(1) == Tq);
  c10::cuda::CUDAGuard guard(q.device());
  C10_CUDA_CHECK(cudaSetDevice(q.device().index()));
  auto stream = at::cuda::getCurrentCUDAStream();
  at::Tensor dq = dq_out.has_value() && dq_out->defined() ? *dq_out : at::empty({Tq, Hq, kD}, q.options());
  at::Tensor dk = dk_out.has_value() && dk_out->defined() ? *dk_out : at::empty({Tk, Hkv, kD}, q.options());
  at::Tensor dv = dv_out.has_value() && dv_out->defined() ? *dv_out : at::empty({Tk, Hkv, kD}, q.options());
  TORCH_CHECK(dq.dim() == 3 && dq.size(0) == Tq && dq.size(1) == Hq && dq.size(2) == kD && dq.stride(2) == 1);
  TORCH_CHECK(dk.dim() == 3 && dk.size(0) == Tk && dk.size(1) == Hkv && dk.size(2) == kD);
  TORCH_CHECK(dv.dim() == 3 && dv.size(0) == Tk && dv.size(1) == Hkv && dv.size(2) == kD);
  if (Tq == 0 || Tk == 0) return {dq, dk, dv};
  const int64_t Tpad = (Tq + 63) / 64 * 64;
  TORCH_CHECK(lse.stride(1) == 1, "flash_bwd: lse rows must be contiguous");
  // rows padded to a multiple of 64 floats (zero filled): the dK/dV kernel fetches 64-row slices with bulk copies
  auto stats = at::zeros({2, Hq, Tpad}, lse.options());
  {
    const int64_t warps = Tq * Hq;
    const int threads = 256;
    flash_delta_kernel<<<(unsigned)((warps * 32 + threads - 1) / threads), threads, 0, stream>>>(
        reinterpret_cast<const __nv_bfloat16*>(o.data_ptr()), reinterpret_cast<const __nv_bfloat16*>(d_o.data_ptr()),
        lse.data_ptr<float>(), (int)lse.stride(0), stats[0].data_ptr<float>(), stats[1].data_ptr<float>(), (int)Tq, (int)Hq,
        (int)Tpad, (float)scale);
    C10_CUDA_KERNEL_LAUNCH_CHECK();
  }
  BwdParams p;
  p.Tq = (int)Tq; p.Tk = (int)Tk; p.Hq = (int)Hq; p.Hkv = (int)Hkv;
  p.causal = causal ? 1 : 0;
  p.causal_offset = (int)causal_offset;
  p.scale = (float)scale;
  p.scale_log2 = (float)(scale * 1.4426950408889634);
  p.kv_first = nullptr;
  if (kv_first.has_value() && kv_first->defined()) {
    TORCH_CHECK(kv_first->is_cuda() && kv_first->scalar_type() == at::kInt && kv_first->numel() == Tq &&
                kv_first->is_contiguous(), "flash_bwd: kv_first must be an int32 [Tq] CUDA tensor");
    p.kv_first = kv_first->data_ptr<int>();
  }
  p.delta = stats[0].data_ptr<float>();
  p.lse = stats[1].data_ptr<float>();
  p.stat_stride = (int)Tpad;
  p.debug = g_flash_debug;
  p.status = flash_status_tensor(q.device()).data_ptr<int>();
  TORCH_CHECK(window >= 0 && (window == 0 || causal), "flash_bwd: a sliding window needs causal attention");
  p.window = (int)window;
  {
    const CUtensorMap tq = make_tmap_thd(q, kBQ), tdo = make_tmap_thd(d_o, kBQ), tk = make_tmap_thd(k, kBN),
                      tv = make_tmap_thd(v, kBN), tdk = make_tmap_thd(dk, kBN), tdv = make_tmap_thd(dv, kBN);
    constexpr uint32_t smem = 2 * kTileBytes + kRing * 2 * kQBytes + kRing * 512 + 1024 + 256;
    static bool attr_set = false;
    if (!attr_set) {
      C10_CUDA_CHECK(cudaFuncSetAttribute(flash_bwd_dkv_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
      attr_set = true;
    }
    const int num_k_tiles = (int)((Tk + kBN - 1) / kBN);
    flash_bwd_dkv_kernel<<<num_k_tiles * (int)Hkv, kThreadsBwd, smem, stream>>>(tq, tdo, tk, tv, tdk, tdv, p);
    C10_CUDA_KERNEL_LAUNCH_CHECK();
  }
  {
    const CUtensorMap tq = make_tmap_thd(q, kBM), tdo = make_tmap_thd(d_o, kBM), tk = make_tmap_thd(k, kBN),
                      tv = make_tmap_thd(v, kBN), tdq = make_tmap_thd(dq, kBM);
    constexpr uint32_t smem = 6 * kTileBytes + 1024 + 256;
    static bool attr_set = false;
    if (!attr_set) {
      C10_CUDA_CHECK(cudaFuncSetAttribute(flash_bwd_dq_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
      attr_set = true;
    }
    const int num_q_tiles = (int)((Tq + kBM - 1) / kBM);
    flash_bwd_dq_kernel<<<num_q_tiles * (int)Hq, kThreadsBwd, smem, stream>>>(tq, tdo, tk, tv, tdq, p);
    C10_CUDA_KERNEL_LAUNCH_CHECK();
  }
  return {dq, dk, dv};
}

// acc_o [T, H, 128] fp32 contiguous, acc_lse [H, T] fp32 (row stride arbitrary), o [T, H, 128] bf16 contiguous,
// lse [H, T] fp32 (row stride arbitrary, e.g. the padded rows flash_fwd returns): merges (o, lse) into the pair.
void attn_merge_(at::Tensor acc_o, at::Tensor acc_lse, const at::Tensor& o, const at::Tensor& lse) {
  using namespace flash;
  TORCH_CHECK(acc_o.is_cuda() && acc_o.scalar_type() == at::kFloat && acc_o.is_contiguous() && acc_o.dim() == 3 &&
              acc_o.size(2) == kD, "attn_merge_: acc_o must be a contiguous fp32 [T, H, 128] tensor");
  TORCH_CHECK(o.scalar_type() == at::kBFloat16 && o.is_contiguous() && o.sizes() == acc_o.sizes());
  const int64_t T = acc_o.size(0), H = acc_o.size(1);
  TORCH_CHECK(acc_lse.scalar_type() == at::kFloat && lse.scalar_type() == at::kFloat && acc_lse.dim() == 2 && lse.dim() == 2 &&
              acc_lse.size(0) == H && acc_lse.size(1) == T && lse.size(0) == H && lse.size(1) == T &&
              acc_lse.stride(1) == 1 && lse.stride(1) == 1);
  if (T * H == 0) return;
  c10::cuda::CUDAGuard guard(acc_o.device());
  const int64_t warps = T * H;
  const int threads = 256;
  attn_merge_kernel<<<(unsigned)((warps * 32 + threads - 1) / threads), threads, 0, at::cuda::getCurrentCUDAStream()>>>(
      acc_o.data_ptr<float>(), acc_lse.data_ptr<float>(), reinterpret_cast<const __nv_bfloat16*>(o.data_ptr()),
      lse.data_ptr<float>(), (int)T, (int)H, (int)acc_lse.stride(0), (int)lse.stride(0));
  C10_CUDA_KERNEL_LAUNCH_CHECK();
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
