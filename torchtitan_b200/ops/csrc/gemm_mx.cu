// MXFP8 block-scaled GEMM: C[M,N] (bf16) = (A . diag-block scales) (B . scales)^T with e4m3 elements and
// one e8m0 scale per 32 K-elements, on tcgen05.mma.kind::mxf8f6f4.block_scale.
//
// A [M, K] and B [N, K] are K-major e4m3 bytes.  Scale factors come in the tiled layout the tensor
// core consumes: for every tile of 128 rows x 128 K-elements (4 scale blocks) one 512-byte atom,
// atoms ordered row-tile major; inside an atom the scale of (row r, block b) sits at byte
// (r % 32) * 16 + (r / 32) * 4 + b.  One atom is a 32-row x 16-byte matrix that tcgen05.cp copies
// into tensor memory, replicated into the four 32-lane quarters ("32x128b.warpx4"); the MMA of a
// lane quarter then finds its rows' scales in its own copy.
//
// Kernel shape: one CTA per 128 x 128 tile (persistent), K step 128 (four MMAs of K = 32 per stage,
// which select scale byte 0..3 of the staged atom through the instruction descriptor), 5-stage TMA
// pipeline (A 16 KB + B 16 KB + scales 1 KB per stage), two TMEM accumulators of 128 columns and
// 8 columns of scale factors per stage.  Roles and the bounded waits are those of the bf16 GEMM.
#include <ATen/ATen.h>
#include <cstdlib>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <cuda.h>

#include "common.cuh"
#include "tc.cuh"

namespace tb200 {
namespace gemm_mx {

using namespace tc;

constexpr int BM = 128, BN = 128, BK = 128;      // BK in elements = bytes
constexpr int kStages = 5;
constexpr int kThreads = 192;
constexpr uint32_t kABytes = BM * BK, kBBytes = BN * BK, kSfBytes = 512;
constexpr uint32_t kStageBytes = kABytes + kBBytes + 2 * kSfBytes;     // 33 KB
constexpr uint32_t kEpiBytes = 4 * 2 * 4096;
constexpr uint32_t kSmemBytes = kStages * kStageBytes + kEpiBytes + 1024 + 256;
constexpr uint32_t kAccCols = 2 * BN;            // two accumulators
constexpr uint32_t kSfColBase = kAccCols;        // 8 scale columns per stage behind the accumulators

struct Params {
  int M, N, K;
  const uint8_t* sfa;     // tiled scales of A: [ceil(M/128)][K/128][512]
  const uint8_t* sfb;     // tiled scales of B
  int* status;
  int debug;              // timing switches: 1 = no loads (barriers only), 2 = no scale copies
  // grouped forms (one-CTA kernel).  mode 1: rows of A / C are grouped (padded expert-major layout,
  // every group starts on a multiple of 128), group g multiplies with rows [g * b_group_rows, ...)
  // of B.  mode 2: the contraction dimension is grouped (weight gradients): group g contracts
  // columns [offs[g], offs[g+1]) of A and B and writes rows [g * M, (g + 1) * M) of C.
  int group_mode;
  int num_groups;
  int b_group_rows;
  const int* group_offs;  // [num_groups + 1], multiples of 128
};

// Instruction descriptor of the block-scaled kinds: e4m3 x e4m3, ue8m0 scales, fp32 accumulate.
__host__ __device__ constexpr uint32_t make_idesc_mx(int m, int n, uint32_t a_sf_id, uint32_t b_sf_id) {
  return (b_sf_id << 4) | (0u << 7) | (0u << 10) | (0u << 15) | (0u << 16) | ((uint32_t)(n >> 3) << 17) | (1u << 23) |
         ((uint32_t)(m >> 4) << 24) | (a_sf_id << 29);
}

// Shared-memory descriptor of a 32-row x 16-byte scale atom (no swizzle: 8-row groups 128 B apart).
__device__ __forceinline__ uint64_t make_sf_desc(uint32_t saddr) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr & 0x3FFFFu) >> 4);
  d |= (uint64_t)((16u >> 4) & 0x3FFFu) << 16;
  d |= (uint64_t)((128u >> 4) & 0x3FFFu) << 32;
  d |= (uint64_t)1 << 46;
  return d;
}

__device__ __forceinline__ void tmem_cp_sf(uint32_t taddr, uint64_t sdesc) {
  asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(sdesc) : "memory");
}

__device__ __forceinline__ void umma_mxf8(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t sfa,
                                          uint32_t sfb, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %6, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale.scale_vec::1X [%0], %1, %2, %3, [%4], [%5], p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(sfa), "r"(sfb), "r"(accumulate)
      : "memory");
}

__global__ void __launch_bounds__(kThreads, 1)
gemm_mxfp8_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                  const __grid_constant__ CUtensorMap tmap_c, const Params p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* gen_base = smem_raw + (base - raw);
  const uint32_t epi_base = base + kStages * kStageBytes;
  const uint32_t bar_base = epi_base + kEpiBytes;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (kStages + s); };
  auto tfull_bar = [&](int a) { return bar_base + 8u * (2 * kStages + a); };
  auto tempty_bar = [&](int a) { return bar_base + 8u * (2 * kStages + 2 + a); };
  uint32_t* tmem_ptr_smem = reinterpret_cast<uint32_t*>(gen_base + kStages * kStageBytes + kEpiBytes + 8 * (2 * kStages + 4));
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_ptr_smem + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int num_m = (p.M + BM - 1) / BM, num_n = (p.N + BN - 1) / BN;
  const int num_tiles = num_m * num_n;
  const int num_kb = (p.K + BK - 1) / BK;
  constexpr int kGroupM = 16;
  auto tile_coord = [&](int t, int& tm, int& tn) {
    const int per_group = kGroupM * num_n;
    const int g = t / per_group;
    const int first = g * kGroupM;
    const int gsz = min(kGroupM, num_m - first);
    const int r = t - g * per_group;
    tm = first + r % gsz;
    tn = r / gsz;
  };

  // Every role derives the same description of a tile (and skips the same tiles).
  struct TileInfo { int skip, tm, tn, a_tile, b_tile, kb0, nkb, c_row; };
  const int tiles_per_group = num_m * num_n;
  const int total_tiles = p.group_mode == 2 ? tiles_per_group * p.num_groups : num_tiles;
  auto tile_info = [&](int t) {
    TileInfo ti;
    int e = 0;
    if (p.group_mode == 2) {
      e = t / tiles_per_group;
      t -= e * tiles_per_group;
    }
    tile_coord(t, ti.tm, ti.tn);
    ti.skip = 0;
    ti.a_tile = ti.tm;
    ti.b_tile = ti.tn;
    ti.kb0 = 0;
    ti.nkb = num_kb;
    ti.c_row = ti.tm * BM;
    if (p.group_mode == 1) {
      const int m0 = ti.tm * BM;
      if (m0 >= p.group_offs[p.num_groups]) {
        ti.skip = 1;
      } else {
        int lo = 0, hi = p.num_groups;     // largest g with group_offs[g] <= m0
        while (hi - lo > 1) {
          const int mid = (lo + hi) >> 1;
          if (p.group_offs[mid] <= m0) lo = mid; else hi = mid;
        }
        ti.b_tile = lo * (p.b_group_rows / BN) + ti.tn;
      }
    } else if (p.group_mode == 2) {
      ti.kb0 = p.group_offs[e] / BK;
      ti.nkb = (p.group_offs[e + 1] - p.group_offs[e]) / BK;
      ti.c_row = e * p.M + ti.tm * BM;
    }
    return ti;
  };

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(tfull_bar(a), 1);
      mbar_init(tempty_bar(a), 4);
    }
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_b);
    tma_prefetch_desc(&tmap_c);
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
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
        const TileInfo ti = tile_info(tile);
        if (ti.skip) continue;
        for (int kk = 0; kk < ti.nkb; ++kk, ++it) {
          const int kb = ti.kb0 + kk;
          const int s = it % kStages;
          if (!mbar_wait(empty_bar(s), ((it / kStages) & 1u) ^ 1u, abort_flag)) { ok = false; break; }
          const uint32_t sa = base + s * kStageBytes, sb = sa + kABytes, ssf = sb + kBBytes;
          mbar_expect_tx(full_bar(s), kStageBytes);
          tma_load_2d(sa, &tmap_a, full_bar(s), kb * BK, ti.a_tile * BM);
          tma_load_2d(sb, &tmap_b, full_bar(s), kb * BK, ti.b_tile * BN);
          bulk_load(ssf, p.sfa + ((int64_t)ti.a_tile * num_kb + kb) * kSfBytes, kSfBytes, full_bar(s));
          bulk_load(ssf + kSfBytes, p.sfb + ((int64_t)ti.b_tile * num_kb + kb) * kSfBytes, kSfBytes, full_bar(s));
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      uint32_t it = 0, tcount = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
        const TileInfo ti = tile_info(tile);
        if (ti.skip) continue;
        const int acc = tcount & 1;
        const uint32_t acc_parity = ((tcount >> 1) & 1u) ^ 1u;
        ++tcount;
        if (!mbar_wait(tempty_bar(acc), acc_parity, abort_flag)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        if (ti.nkb == 0) {          // an empty group: nothing to multiply, the epilogue writes zeros
          mbar_arrive(tfull_bar(acc));
          continue;
        }
        for (int kb = 0; kb < ti.nkb; ++kb, ++it) {
          const int s = it % kStages;
          if (!mbar_wait(full_bar(s), (it / kStages) & 1u, abort_flag)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sa = base + s * kStageBytes, sb = sa + kABytes, ssf = sb + kBBytes;
          const uint32_t t_sfa = tmem_base + kSfColBase + s * 8, t_sfb = t_sfa + 4;
          tmem_cp_sf(t_sfa, make_sf_desc(ssf));
          tmem_cp_sf(t_sfb, make_sf_desc(ssf + kSfBytes));
#pragma unroll
          for (int k = 0; k < BK / 32; ++k)
            umma_mxf8(d_tmem, make_desc(sa + k * 32, 16, 1024), make_desc(sb + k * 32, 16, 1024),
                      make_idesc_mx(BM, BN, k, k), t_sfa, t_sfb, (kb | k) != 0 ? 1u : 0u);
          umma_commit(empty_bar(s));
        }
        if (ok) umma_commit(tfull_bar(acc));
      }
    }
  } else {
    const int q = warp & 3;
    uint32_t tcount = 0, sbuf = 0;
    bool ok = true;
    const int c_rows = p.group_mode == 2 ? p.M * p.num_groups : p.M;
    for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
      const TileInfo ti = tile_info(tile);
      if (ti.skip) continue;
      const int acc = tcount & 1;
      const uint32_t acc_parity = (tcount >> 1) & 1u;
      ++tcount;
      const int m0 = ti.c_row, n0 = ti.tn * BN;
      if (!mbar_wait(tfull_bar(acc), acc_parity, abort_flag)) { ok = false; break; }
      tc_fence_after();
      const uint32_t stage0 = epi_base + (uint32_t)(warp - 2) * 8192u;
#pragma unroll 1
      for (int c = 0; c < BN / 64; ++c) {
        uint32_t r0[32], r1[32];
        const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(acc * BN + c * 64);
        if (ti.nkb > 0) {
          tmem_ld32(taddr, r0);
          tmem_ld32(taddr + 32, r1);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int e = 0; e < 32; ++e) r0[e] = r1[e] = 0u;
        }
        if (lane == 0) tma_store_wait_read<1>();
        __syncwarp();
        const uint32_t buf = stage0 + (sbuf ? 4096u : 0u);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          uint32_t w[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int i = (j & 3) * 8 + 2 * e;
            __nv_bfloat162 h = __floats2bfloat162_rn(__uint_as_float(j < 4 ? r0[i] : r1[i]),
                                                      __uint_as_float(j < 4 ? r0[i + 1] : r1[i + 1]));
            w[e] = *reinterpret_cast<uint32_t*>(&h);
          }
          const uint32_t dst = buf + (uint32_t)lane * 128u + (uint32_t)((j ^ (lane & 7)) << 4);
          asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(w[0]), "r"(w[1]), "r"(w[2]), "r"(w[3])
                       : "memory");
        }
        fence_proxy_async_smem();
        __syncwarp();
        const int col0 = n0 + c * 64;
        if (lane == 0 && col0 < p.N && m0 + q * 32 < c_rows) {
          tma_store_2d(&tmap_c, buf, col0, m0 + q * 32);
          tma_store_commit();
        }
        sbuf ^= 1u;
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(tempty_bar(acc));
    }
    if (lane == 0) tma_store_wait<0>();
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
  if (threadIdx.x == 0 && *abort_flag && p.status != nullptr) atomicOr(p.status, kStatusWaitTimedOut);
}

// ---------------------------------------------------------------------------------------------
// CTA-pair form: a cluster of two CTAs (one SM pair) computes a 256 x 256 tile with
// tcgen05.mma.cta_group::2.  Each CTA stages its own 128 rows of A, its own 128 of the tile's 256
// rows of B, the scale atom of its A rows and both scale atoms of B; four warps of each CTA move
// the atoms from shared to tensor memory with tcgen05.st (a tcgen05.cp between the MMAs measured
// 25 % slower: the copy drains the tensor pipe); CTA 0 issues every MMA.  Tensor memory holds ONE 256-column accumulator plus 16 scale columns
// per stage, so the accumulator cannot be double buffered there: eight epilogue warps copy it to
// registers (128 columns of 32 lanes each, packed to bf16), release it at once, and store from
// registers (32 x 32 tiles through a 64B-swizzled staging buffer and TMA) while the MMAs of the next
// tile run.  What limits this kernel is operand feed: without cluster multicast every CTA pulls its
// own 32 KB per K step from L2, so throughput is bytes in flight / L2 latency; hence six stages and a
// small epilogue buffer.
namespace pair {
constexpr int BN2 = 256;                          // columns of the pair tile
constexpr int kPStages = 6;
constexpr int kPThreads = 64 + 8 * 32 + 4 * 32;    // producer, MMA, 8 epilogue warps, 4 scale warps
constexpr uint32_t kPABytes = BM * BK, kPBBytes = (BN2 / 2) * BK;
constexpr uint32_t kDataBytes = kPABytes + kPBBytes;                     // 32 KB per stage (1024-byte multiple)
constexpr uint32_t kSfStage = 3 * kSfBytes;                            // A atom, two B atoms
constexpr uint32_t kPEpiBytes = 8 * 2048;                                // one 32 x 32 bf16 tile per epilogue warp
constexpr uint32_t kSfRegion = (kPStages * kSfStage + 1023u) & ~1023u;   // keeps the swizzled epilogue tiles 1024-byte aligned
constexpr uint32_t kPSmemBytes = kPStages * kDataBytes + kSfRegion + kPEpiBytes + 1024 + 256;
constexpr uint32_t kSfCol0 = BN2;                                      // 16 scale columns per stage
}  // namespace pair

__device__ __forceinline__ void umma_mxf8_pair(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t sfa,
                                               uint32_t sfb, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %6, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::mxf8f6f4.block_scale.scale_vec::1X [%0], %1, %2, %3, [%4], [%5], p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(sfa), "r"(sfb), "r"(accumulate)
      : "memory");
}

__global__ void __launch_bounds__(pair::kPThreads, 1)
gemm_mxfp8_pair_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                       const __grid_constant__ CUtensorMap tmap_c, const __grid_constant__ CUtensorMap tmap_sfa,
                       const __grid_constant__ CUtensorMap tmap_sfb, const Params p) {
  using namespace pair;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* gen_base = smem_raw + (base - raw);
  const uint32_t sf_base = base + kPStages * kDataBytes;
  const uint32_t epi_base = sf_base + kSfRegion;
  const uint32_t bar_base = epi_base + kPEpiBytes;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (kPStages + s); };
  auto sf_full_bar = [&](int s) { return bar_base + 8u * (2 * kPStages + s); };      // this CTA's scale atoms landed
  auto sf_ready_bar = [&](int s) { return bar_base + 8u * (3 * kPStages + s); };     // scales of both CTAs are in TMEM
  const uint32_t tfull_bar = bar_base + 8u * (4 * kPStages), tempty_bar = tfull_bar + 8u;
  uint32_t* tmem_ptr_smem = reinterpret_cast<uint32_t*>(gen_base + (bar_base - base) + 8 * (4 * kPStages + 2));
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_ptr_smem + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t cta_rank = cluster_ctarank();
  const int unit = (int)(blockIdx.x >> 1), num_units = (int)(gridDim.x >> 1);
  constexpr int kTileM = 2 * BM;
  const int num_m = (p.M + kTileM - 1) / kTileM, num_n = (p.N + BN2 - 1) / BN2;
  const int num_tiles = num_m * num_n;
  const int num_kb = (p.K + BK - 1) / BK;
  constexpr int kGroupM = 8;
  auto tile_coord = [&](int t, int& tm, int& tn) {
    const int per_group = kGroupM * num_n;
    const int g = t / per_group;
    const int first = g * kGroupM;
    const int gsz = min(kGroupM, num_m - first);
    const int r = t - g * per_group;
    tm = first + r % gsz;
    tn = r / gsz;
  };

  if (threadIdx.x == 0) {
    for (int s = 0; s < kPStages; ++s) {
      mbar_init(full_bar(s), 2);       // one arrive.expect_tx per producing CTA
      mbar_init(empty_bar(s), 1);
      mbar_init(sf_full_bar(s), 1);
      mbar_init(sf_ready_bar(s), 8);   // four scale warps of each CTA
    }
    mbar_init(tfull_bar, 1);
    mbar_init(tempty_bar, 16);         // eight epilogue warps of each CTA
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_b);
    tma_prefetch_desc(&tmap_c);
    tma_prefetch_desc(&tmap_sfa);
    tma_prefetch_desc(&tmap_sfb);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_ptr_smem), 512);     // the whole TMEM: both CTAs get base column 0
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_ptr_smem;

  if (warp == 0) {
    if (lane == 0) {
      uint32_t s = 0, phase = 1;
      bool ok = true;
      const uint32_t fb0 = mapa(full_bar(0), 0);                       // CTA 0 counts the bytes of both
      for (int tile = unit; tile < num_tiles && ok; tile += num_units) {
        int tm, tn;
        tile_coord(tile, tm, tn);
        const int mt = tm * 2 + (int)cta_rank;                       // 128-row tile of A staged here
        const int b_row = tn * BN2 + (int)cta_rank * (BN2 / 2);
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait_cluster(empty_bar(s), phase, abort_flag)) { ok = false; break; }
          const uint32_t sa = base + s * kDataBytes, sb = sa + kPABytes, ssf = sf_base + s * kSfStage;
          const uint32_t fb = fb0 + 8u * s;
          if (p.debug & 1) {
            mbar_arrive_cluster(fb);
            mbar_arrive(sf_full_bar(s));
          } else {
            mbar_expect_tx_cluster(fb, kDataBytes);
            tma_load_2d_pair(sa, &tmap_a, fb, kb * BK, mt * BM);
            tma_load_2d_pair(sb, &tmap_b, fb, kb * BK, b_row);
            mbar_expect_tx(sf_full_bar(s), kSfStage);                  // scales: this CTA's own barrier
            tma_load_3d(ssf, &tmap_sfa, sf_full_bar(s), 0, kb, mt);
            tma_load_3d(ssf + kSfBytes, &tmap_sfb, sf_full_bar(s), 0, kb, tn * 2);
          }
          if (++s == kPStages) { s = 0; phase ^= 1u; }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && cta_rank == 0) {
      // One thread feeds a tensor pipe that retires a stage in ~512 cycles, so the loop is kept short:
      // descriptors are a constant high word and a low word that advances by adds, the stage index
      // and barrier phase are counters (no division), the instruction descriptors are constants.
      const uint32_t desc_hi = (1024u >> 4) | (1u << 14) | (2u << 29);        // SBO 1024 B, version 1, 128B swizzle
      const uint32_t a_lo0 = ((base & 0x3FFFFu) >> 4) | (1u << 16);           // LBO 16 B
      uint32_t s = 0, phase = 0, tcount = 0;
      bool ok = true;
      for (int tile = unit; tile < num_tiles && ok; tile += num_units, ++tcount) {
        if (!mbar_wait_cluster(tempty_bar, (tcount & 1u) ^ 1u, abort_flag)) { ok = false; break; }
        tc_fence_after();
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait_cluster(full_bar(s), phase, abort_flag) || !mbar_wait_cluster(sf_ready_bar(s), phase, abort_flag)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t a_lo = a_lo0 + s * (kDataBytes >> 4), b_lo = a_lo + (kPABytes >> 4);
          const uint32_t t_sfa = tmem_base + kSfCol0 + s * 16, t_sfb = t_sfa + 4;
#pragma unroll
          for (int k = 0; k < BK / 32; ++k)
            umma_mxf8_pair(tmem_base, ((uint64_t)desc_hi << 32) | (a_lo + 2u * k), ((uint64_t)desc_hi << 32) | (b_lo + 2u * k),
                           make_idesc_mx(kTileM, BN2, k, k), t_sfa, t_sfb, k != 0 ? 1u : (uint32_t)(kb != 0));
          umma_commit_pair(empty_bar(s), 3);
          if (++s == kPStages) { s = 0; phase ^= 1u; }
        }
        if (ok) umma_commit_pair(tfull_bar, 3);
      }
    }
  } else if (warp >= 10) {
    // ------------------------------------------------------------- scale warps (every CTA)
    // Each of the four warps writes the stage's scale atoms (A: 4 columns, B: 8 columns) into its own
    // 32-lane quarter of this CTA's tensor memory: the layout a tcgen05.cp "32x128b.warpx4" would
    // produce, without putting a copy between the MMAs of the tensor pipe.
    const uint32_t q = (uint32_t)(warp & 3);
    const uint32_t ready_leader = mapa(sf_ready_bar(0), 0);
    uint32_t it = 0;
    bool ok = true;
    for (int tile = unit; tile < num_tiles && ok; tile += num_units) {
      for (int kb = 0; kb < num_kb; ++kb, ++it) {
        const int s = it % kPStages;
        if (!mbar_wait(sf_full_bar(s), (it / kPStages) & 1u, abort_flag)) { ok = false; break; }
        if (!(p.debug & 2)) {
          const uint32_t ssf = sf_base + s * kSfStage + (uint32_t)lane * 16u;
          uint32_t a[4], b[8];
          asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(a[0]), "=r"(a[1]), "=r"(a[2]), "=r"(a[3]) : "r"(ssf));
          asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];"
                       : "=r"(b[0]), "=r"(b[1]), "=r"(b[2]), "=r"(b[3]) : "r"(ssf + kSfBytes));
          asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];"
                       : "=r"(b[4]), "=r"(b[5]), "=r"(b[6]), "=r"(b[7]) : "r"(ssf + 2 * kSfBytes));
          const uint32_t t = tmem_base + ((q * 32u) << 16) + kSfCol0 + (uint32_t)s * 16u;
          asm volatile("tcgen05.st.sync.aligned.32x32b.x4.b32 [%0], {%1, %2, %3, %4};"
                       ::"r"(t), "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]) : "memory");
          tmem_st8(t + 4, b);
          tmem_st_wait();
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(ready_leader + 8u * s);
      }
    }
  } else {
    const int q = warp & 3;                 // TMEM lane quarter of this warp
    const int h = (warp - 2) >> 2;          // column half of the tile
    uint32_t tcount = 0;
    bool ok = true;
    const uint32_t te_leader = mapa(tempty_bar, 0);
    const uint32_t buf = epi_base + (uint32_t)(warp - 2) * 2048u;
    for (int tile = unit; tile < num_tiles && ok; tile += num_units, ++tcount) {
      int tm, tn;
      tile_coord(tile, tm, tn);
      const int m0 = tm * kTileM + (int)cta_rank * BM + q * 32, n0 = tn * BN2 + h * 128;
      if (!mbar_wait_cluster(tfull_bar, tcount & 1u, abort_flag)) { ok = false; break; }
      tc_fence_after();
      uint32_t packed[64];                  // 128 columns of this lane's row as bf16 pairs
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t r[32];
        tmem_ld32(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(h * 128 + c * 32), r);
        tmem_ld_wait();
#pragma unroll
        for (int e = 0; e < 16; ++e) {
          __nv_bfloat162 v = __floats2bfloat162_rn(__uint_as_float(r[2 * e]), __uint_as_float(r[2 * e + 1]));
          packed[c * 16 + e] = *reinterpret_cast<uint32_t*>(&v);
        }
      }
      // the accumulator is free again: the MMAs of the next tile may overwrite it
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(te_leader);
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        if (lane == 0) tma_store_wait_read<0>();   // the previous store has read the staging tile
        __syncwarp();
#pragma unroll
        for (int j = 0; j < 4; ++j) {              // 64-byte rows, 16-byte chunks XOR-swizzled by (row / 2) % 4
          const uint32_t dst = buf + (uint32_t)lane * 64u + (uint32_t)((j ^ ((lane >> 1) & 3)) << 4);
          const int e = c * 16 + j * 4;
          asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(packed[e]), "r"(packed[e + 1]),
                       "r"(packed[e + 2]), "r"(packed[e + 3])
                       : "memory");
        }
        fence_proxy_async_smem();
        __syncwarp();
        const int col0 = n0 + c * 32;
        if (lane == 0 && col0 < p.N && m0 < p.M) {
          tma_store_2d(&tmap_c, buf, col0, m0);
          tma_store_commit();
        }
      }
    }
    if (lane == 0) tma_store_wait<0>();
  }

  tc_fence_before();
  __syncthreads();
  cluster_sync();      // neither CTA frees its TMEM or leaves while the other can still issue MMAs
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
  if (threadIdx.x == 0 && *abort_flag && p.status != nullptr) atomicOr(p.status, kStatusWaitTimedOut);
}

}  // namespace gemm_mx

static CUtensorMap make_tmap_2d_t(const void* ptr, CUtensorMapDataType dt, uint64_t esz, uint64_t inner, uint64_t outer,
                                  uint32_t box_inner, uint32_t box_outer,
                                  CUtensorMapSwizzle swizzle = CU_TENSOR_MAP_SWIZZLE_128B) {
  CUtensorMap map;
  const cuuint64_t dims[2] = {inner, outer};
  const cuuint64_t strides[1] = {inner * esz};
  const cuuint32_t box[2] = {box_inner, box_outer};
  const cuuint32_t elem[2] = {1, 1};
  const CUresult r = cuTensorMapEncodeTiled(&map, dt, 2, const_cast<void*>(ptr), dims, strides, box, elem,
                                            CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle,
                                            CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  TORCH_CHECK(r == CUDA_SUCCESS, "cuTensorMapEncodeTiled (mxfp8 gemm) failed with code ", (int)r);
  return map;
}

// Scale atoms as a 3-D tensor [row tile][K tile][128 words] for the pair kernel's tile loads.
static CUtensorMap make_tmap_sf(const void* ptr, uint64_t row_tiles, uint64_t k_tiles, uint32_t box_tiles) {
  CUtensorMap map;
  const cuuint64_t dims[3] = {128, k_tiles, row_tiles};
  const cuuint64_t strides[2] = {512, 512 * k_tiles};
  const cuuint32_t box[3] = {128, 1, box_tiles};
  const cuuint32_t elem[3] = {1, 1, 1};
  const CUresult r = cuTensorMapEncodeTiled(&map, CU_TENSOR_MAP_DATA_TYPE_UINT32, 3, const_cast<void*>(ptr), dims, strides,
                                            box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
                                            CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  TORCH_CHECK(r == CUDA_SUCCESS, "cuTensorMapEncodeTiled (mxfp8 scales) failed with code ", (int)r);
  return map;
}

static int g_mx_debug = 0;
// Timing diagnostics that make the kernel skip part of its work (results are garbage by design).
// Refused unless the process was started with TB200_KERNEL_TIMING_DEBUG=1, so that no training
// job can switch them on by accident.
void gemm_mx_set_debug(int64_t v) {
  TORCH_CHECK(v == 0 || std::getenv("TB200_KERNEL_TIMING_DEBUG") != nullptr,
              "gemm_mx_set_debug: set TB200_KERNEL_TIMING_DEBUG=1 in the environment to enable the timing switches");
  g_mx_debug = (int)v;
}
static int g_mx_variant = 0;   // 0: by shape, 1: one CTA per tile, 2: CTA pairs
void gemm_mx_set_variant(int64_t v) {
  TORCH_CHECK(v >= 0 && v <= 2, "gemm_mx_set_variant: 0 (auto), 1 (single CTA) or 2 (CTA pair)");
  g_mx_variant = (int)v;
}

int64_t gemm_status(bool clear);

// a [M, K], b [N, K]: e4m3 bytes (uint8), K a multiple of 128; sfa / sfb: tiled e8m0 scales
// (`mxfp8_quantize_tiled`); returns C [M, N] bf16 = dequant(a) . dequant(b)^T.
at::Tensor gemm_mxfp8(const at::Tensor& a, const at::Tensor& sfa, const at::Tensor& b, const at::Tensor& sfb) {
  using namespace gemm_mx;
  TORCH_CHECK(a.is_cuda() && b.is_cuda() && a.scalar_type() == at::kByte && b.scalar_type() == at::kByte);
  TORCH_CHECK(a.dim() == 2 && b.dim() == 2 && a.is_contiguous() && b.is_contiguous() && a.size(1) == b.size(1));
  const int64_t M = a.size(0), N = b.size(0), K = a.size(1);
  TORCH_CHECK(K % BK == 0 && N % 8 == 0, "gemm_mxfp8: K must be a multiple of 128 and N of 8");
  const int64_t kt = K / BK;
  TORCH_CHECK(sfa.is_cuda() && sfa.scalar_type() == at::kByte && sfa.is_contiguous() &&
              sfa.numel() == (M + 127) / 128 * kt * 512, "gemm_mxfp8: sfa has the wrong size");
  TORCH_CHECK(sfb.is_cuda() && sfb.scalar_type() == at::kByte && sfb.is_contiguous() &&
              sfb.numel() == (N + 127) / 128 * kt * 512, "gemm_mxfp8: sfb has the wrong size");
  c10::cuda::CUDAGuard guard(a.device());
  C10_CUDA_CHECK(cudaSetDevice(a.device().index()));
  auto c = at::empty({M, N}, a.options().dtype(at::kBFloat16));
  if (M == 0 || N == 0) return c;
  const CUtensorMap ta = make_tmap_2d_t(a.data_ptr(), CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, K, M, BK, BM);
  const CUtensorMap tb = make_tmap_2d_t(b.data_ptr(), CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, K, N, BK, BN);
  const CUtensorMap tcm = make_tmap_2d_t(c.data_ptr(), CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, N, M, 64, 32);
  Params p;
  p.M = (int)M; p.N = (int)N; p.K = (int)K;
  p.sfa = sfa.data_ptr<uint8_t>();
  p.sfb = sfb.data_ptr<uint8_t>();
  static at::Tensor status;
  if (!status.defined()) status = at::zeros({1}, a.options().dtype(at::kInt));
  p.status = status.data_ptr<int>();
  p.debug = g_mx_debug;
  p.group_mode = 0; p.num_groups = 0; p.b_group_rows = 0; p.group_offs = nullptr;
  const bool use_pair = g_mx_variant == 2 || (g_mx_variant == 0 && M >= 512 && N >= 256);
  if (use_pair) {
    const CUtensorMap tb2 = make_tmap_2d_t(b.data_ptr(), CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, K, N, BK, pair::BN2 / 2);
    const CUtensorMap tc2 = make_tmap_2d_t(c.data_ptr(), CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, N, M, 32, 32,
                                           CU_TENSOR_MAP_SWIZZLE_64B);
    const CUtensorMap tsa = make_tmap_sf(sfa.data_ptr(), (M + 127) / 128, kt, 1);
    const CUtensorMap tsb = make_tmap_sf(sfb.data_ptr(), (N + 127) / 128, kt, 2);
    static bool pair_attr_set = false;
    if (!pair_attr_set) {
      C10_CUDA_CHECK(cudaFuncSetAttribute(gemm_mxfp8_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                          pair::kPSmemBytes));
      pair_attr_set = true;
    }
    const int tiles = (int)(((M + 255) / 256) * ((N + pair::BN2 - 1) / pair::BN2));
    cudaLaunchConfig_t cfg = {};
    cfg.blockDim = dim3(pair::kPThreads);
    cfg.dynamicSmemBytes = pair::kPSmemBytes;
    cfg.stream = at::cuda::getCurrentCUDAStream();
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    static int max_pairs = 0;
    if (max_pairs == 0) {
      cfg.gridDim = dim3(num_sms() & ~1);
      int n = 0;
      C10_CUDA_CHECK(cudaOccupancyMaxActiveClusters(&n, gemm_mxfp8_pair_kernel, &cfg));
      max_pairs = std::max(1, std::min(n, num_sms() / 2));
    }
    cfg.gridDim = dim3(2 * std::min(tiles, max_pairs));
    C10_CUDA_CHECK(cudaLaunchKernelEx(&cfg, gemm_mxfp8_pair_kernel, ta, tb2, tc2, tsa, tsb, p));
    return c;
  }
  static bool attr_set = false;
  if (!attr_set) {
    C10_CUDA_CHECK(cudaFuncSetAttribute(gemm_mxfp8_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes));
    attr_set = true;
  }
  const int tiles = (int)(((M + BM - 1) / BM) * ((N + BN - 1) / BN));
  gemm_mxfp8_kernel<<<std::min(tiles, num_sms()), kThreads, kSmemBytes, at::cuda::getCurrentCUDAStream()>>>(ta, tb, tcm, p);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  return c;
}

// Grouped MXFP8 GEMMs of the expert layers (one-CTA kernel, 128 x 128 tiles).
//   mode 1: a [R, K] rows in the padded expert-major layout (offs[E + 1], multiples of 128),
//           b [E * N, K] the stacked expert matrices (N % 128 == 0)  ->  C [R, N];
//           rows at or beyond offs[E] are not written.
//   mode 2: a [M, R], b [N, R] with the contraction dimension R grouped by offs
//           (M % 128 == 0)  ->  C [E * M, N], zeros for an empty group.
at::Tensor gemm_mxfp8_grouped(const at::Tensor& a, const at::Tensor& sfa, const at::Tensor& b, const at::Tensor& sfb,
                              const at::Tensor& offs, int64_t mode) {
  using namespace gemm_mx;
  TORCH_CHECK(mode == 1 || mode == 2, "gemm_mxfp8_grouped: mode 1 (rows grouped) or 2 (contraction grouped)");
  TORCH_CHECK(a.is_cuda() && b.is_cuda() && a.scalar_type() == at::kByte && b.scalar_type() == at::kByte);
  TORCH_CHECK(a.dim() == 2 && b.dim() == 2 && a.is_contiguous() && b.is_contiguous() && a.size(1) == b.size(1));
  TORCH_CHECK(offs.is_cuda() && offs.scalar_type() == at::kInt && offs.is_contiguous() && offs.numel() >= 2);
  const int64_t E = offs.numel() - 1;
  const int64_t K = a.size(1);
  TORCH_CHECK(K % BK == 0, "gemm_mxfp8_grouped: the contraction dimension must be a multiple of 128");
  const int64_t kt = K / BK;
  int64_t M, N, c_rows;
  if (mode == 1) {
    TORCH_CHECK(b.size(0) % E == 0 && (b.size(0) / E) % BN == 0, "gemm_mxfp8_grouped: b must stack E matrices of N % 128 == 0 rows");
    M = a.size(0); N = b.size(0) / E; c_rows = M;
  } else {
    TORCH_CHECK(a.size(0) % BM == 0 && b.size(0) % 8 == 0, "gemm_mxfp8_grouped: mode 2 needs M % 128 == 0 and N % 8 == 0");
    M = a.size(0); N = b.size(0); c_rows = E * M;
  }
  TORCH_CHECK(sfa.is_cuda() && sfa.scalar_type() == at::kByte && sfa.is_contiguous() &&
              sfa.numel() == (a.size(0) + 127) / 128 * kt * 512, "gemm_mxfp8_grouped: sfa has the wrong size");
  TORCH_CHECK(sfb.is_cuda() && sfb.scalar_type() == at::kByte && sfb.is_contiguous() &&
              sfb.numel() == (b.size(0) + 127) / 128 * kt * 512, "gemm_mxfp8_grouped: sfb has the wrong size");
  c10::cuda::CUDAGuard guard(a.device());
  C10_CUDA_CHECK(cudaSetDevice(a.device().index()));
  // mode 1 leaves the rows behind the last group untouched: they read as zeros
  auto c = mode == 1 ? at::zeros({c_rows, N}, a.options().dtype(at::kBFloat16))
                     : at::empty({c_rows, N}, a.options().dtype(at::kBFloat16));
  if (c_rows == 0 || N == 0) return c;
  const CUtensorMap ta = make_tmap_2d_t(a.data_ptr(), CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, K, a.size(0), BK, BM);
  const CUtensorMap tb = make_tmap_2d_t(b.data_ptr(), CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, K, b.size(0), BK, BN);
  const CUtensorMap tcm = make_tmap_2d_t(c.data_ptr(), CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, N, c_rows, 64, 32);
  Params p;
  p.M = (int)M; p.N = (int)N; p.K = (int)K;
  p.sfa = sfa.data_ptr<uint8_t>();
  p.sfb = sfb.data_ptr<uint8_t>();
  static at::Tensor status;
  if (!status.defined()) status = at::zeros({1}, a.options().dtype(at::kInt));
  p.status = status.data_ptr<int>();
  p.debug = 0;
  p.group_mode = (int)mode; p.num_groups = (int)E; p.b_group_rows = (int)N; p.group_offs = offs.data_ptr<int>();
  static bool attr_set = false;
  if (!attr_set) {
    C10_CUDA_CHECK(cudaFuncSetAttribute(gemm_mxfp8_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes));
    attr_set = true;
  }
  const int64_t tiles = ((M + BM - 1) / BM) * ((N + BN - 1) / BN) * (mode == 2 ? E : 1);
  gemm_mxfp8_kernel<<<(int)std::min<int64_t>(tiles, num_sms()), kThreads, kSmemBytes, at::cuda::getCurrentCUDAStream()>>>(
      ta, tb, tcm, p);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  return c;
}

}  // namespace tb200
