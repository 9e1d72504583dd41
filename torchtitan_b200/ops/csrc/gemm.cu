// bf16 GEMM on the 5th-generation tensor cores: tcgen05.mma with TMEM accumulators,
// operands staged by TMA into 128B-swizzled shared memory, persistent warp-specialised CTAs.
//
//   mode 0 (NT): C[M,N] = A[M,K] . B[N,K]^T      forward of a linear layer
//   mode 1 (NN): C[M,N] = A[M,K] . B[K,N]        input gradient
//   mode 2 (TN): C[M,N] = A[K,M]^T . B[K,N]      weight gradient
// `accumulate` adds the product, rounded to bf16, to the existing C with a TMA reduce-add.
//
// Two instantiations of one kernel body:
//   kCta = 1 : one CTA per SM computes a 128 x 256 tile, 4-stage TMA pipeline (48 KB per stage).
//   kCta = 2 : a cluster of two CTAs (one SM pair) computes a 256 x 256 tile with
//              tcgen05.mma.cta_group::2.  Each CTA stages its own 128 rows of A and its own 128
//              rows (columns of C) of B, so a stage is 32 KB per CTA and the pipeline has 6
//              stages; the B traffic per SM halves.  The MMA is issued by CTA 0 only and writes the
//              accumulator rows of both CTAs' TMEM; both CTAs run a producer and an epilogue.
// Roles inside a CTA:
//   warp 0      : TMA producer (one elected lane)
//   warp 1      : allocates TMEM, issues tcgen05.mma (one elected lane), commits to mbarriers
//   warps 2..5  : epilogue; each warp owns the 32 TMEM lanes of its quarter (warp_id % 4),
//                 reads the fp32 accumulator with tcgen05.ld, converts and stores bf16
// The 512 TMEM columns hold two 128 x 256 fp32 accumulators, so the epilogue of tile i
// overlaps the main loop of tile i+1.
//
// Tiles are visited in groups of kGroupRows rows of C (about 2048) so that the CTAs that run
// at the same time share A and B panels in L2.
//
// Operand layouts.  K-major operands ([rows, K] row-major) are loaded as boxes of 64 K-elements
// (128 B) x rows; MN-major operands ([K, cols] row-major) as boxes of 64 columns (128 B) x 64
// K-rows, one box per 64 columns.  Both use the 128-byte swizzle, which is what the shared
// memory matrix descriptors describe.
//
// Every mbarrier wait is bounded: after a fixed number of polls the waiter raises an abort flag
// in shared memory, all roles leave their loops, TMEM is freed and the kernel sets bit
// kStatusWaitTimedOut in the status word.  TMA loads are plain tile loads: the CTA pair uses the
// cta_group::2 form only so that both CTAs can report bytes to the barrier of CTA 0.
#include <ATen/ATen.h>
#include <cstdlib>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <cuda.h>

#include "common.cuh"
#include "tc.cuh"

namespace tb200 {

namespace gemm {

using namespace tc;

constexpr int BM = 128;   // rows of C per CTA
constexpr int BN = 256;   // columns of C per tile
constexpr int BK = 64;
constexpr int UMMA_K = 16;
constexpr int kThreads = 192;
constexpr uint32_t kTmemCols = 512;
constexpr int kGroupRows = 2048;

template <int kCta>
struct Cfg {
  static constexpr int kStages = kCta == 1 ? 4 : 6;
  static constexpr int kBRows = BN / kCta;                 // rows of B staged by one CTA
  static constexpr uint32_t kABytes = BM * BK * 2;         // 16 KB
  static constexpr uint32_t kBBytes = kBRows * BK * 2;     // 32 KB or 16 KB
  static constexpr uint32_t kStageBytes = kABytes + kBBytes;
  static constexpr uint32_t kEpiBytes = 4 * 2 * 4096;      // per epilogue warp: two 32-row x 128 B staging tiles
  static constexpr uint32_t kSmemBytes = kStages * kStageBytes + kEpiBytes + 1024 /*alignment slack*/ + 256 /*barriers*/;
};

struct Params {
  int M, N, K;
  int a_mn_major;  // A is stored [K, M]
  int b_mn_major;  // B is stored [K, N]
  // MN-major operand described by a 3-D tensor map [MN / 64][K][64]: one load brings all 64-column boxes of a stage
  int a_mn3d, b_mn3d;
  int accumulate;
  int debug;       // bit 0: no TMA loads (MMA issue rate on stale shared memory), bit 1: no stores
  __nv_bfloat16* C;
  int* status;
  // Grouped forms (rows sorted by group, e.g. tokens sorted by expert).  group_offs[g] is the first
  // row of group g, group_offs[num_groups] the number of valid rows; every offset is a multiple of
  // the row tile, so no tile straddles two groups.
  //   group_mode 1: rows of A and C are grouped, B holds one matrix per group (b_group_rows rows each)
  //   group_mode 2: the K dimension (rows of A and B in TN mode) is grouped, C holds one M x N matrix per group
  const int* group_offs;
  int num_groups;
  int group_mode;
  int b_group_rows;
  int c_rows;       // rows of the 2-D view of C
  // ---- communication fused into the kernel (kComm instantiation only)
  // All-gather -> GEMM: A is this rank's gather buffer [ranks * shard_rows, K].  The rank's own
  // shard is already there; 128 extra threads per CTA pull the other shards from the peers' gather
  // buffers (plain 16-byte peer loads over NVLink, local stores) in blocks of 128 rows and publish
  // one flag per block; the TMA producer waits for the flag of a row block before it loads it,
  // and row tiles are visited starting with the local shard, in the order the blocks arrive.
  // GEMM -> reduce-scatter: the epilogue stores each tile into the staging buffer of the rank that
  // owns those rows (slot = this rank) with TMA stores to peer memory; rows of the next ranks first.
  uint32_t* a_flags;          // [ranks * shard_rows / 128], value = epoch once the block is local
  const uint32_t* a_epoch;     // device counter: the value it holds when the kernel starts is this launch's epoch
                               // (kept on the device so that a replayed CUDA graph sees a fresh epoch each time)
  int m_rotate;               // row tiles are visited from this tile index on (wrapping)
  int gather_ranks, gather_rank, gather_shard_rows, gather_row_bytes;
  const uint8_t* gather_src[8];
  uint8_t* gather_dst;
  int scatter_ranks, scatter_rank, scatter_shard_rows;
};

struct CommMaps {
  CUtensorMap m[8];           // staging buffers of the ranks (GEMM -> reduce-scatter)
};

constexpr int kCommThreads = 128;

struct Tile {
  int skip, m_base, n0, c_row, b_row_off, k_beg, nkb;
};

template <int kCta, bool kComm>
__global__ void __launch_bounds__(kThreads + (kComm ? kCommThreads : 0), 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                 const __grid_constant__ CUtensorMap tmap_c, const __grid_constant__ CommMaps cmaps, const Params p) {
  using C_ = Cfg<kCta>;
  constexpr int kStages = C_::kStages;
  constexpr uint32_t kABytes = C_::kABytes, kStageBytes = C_::kStageBytes;
  extern __shared__ uint8_t smem_raw[];
  // stage buffers need 1024-byte alignment for the 128B swizzle atoms
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* gen_base = smem_raw + (base - raw);
  const uint32_t epi_base = base + kStages * kStageBytes;
  const uint32_t bar_base = epi_base + C_::kEpiBytes;
  // barrier layout: full[kStages], empty[kStages], tmem_full[2], tmem_empty[2], then tmem ptr, abort flag
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (kStages + s); };
  auto tfull_bar = [&](int a) { return bar_base + 8u * (2 * kStages + a); };
  auto tempty_bar = [&](int a) { return bar_base + 8u * (2 * kStages + 2 + a); };
  uint32_t* tmem_ptr_smem =
      reinterpret_cast<uint32_t*>(gen_base + kStages * kStageBytes + C_::kEpiBytes + 8 * (2 * kStages + 4));
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_ptr_smem + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t cta_rank = kCta == 1 ? 0u : cluster_ctarank();
  const int unit = kCta == 1 ? (int)blockIdx.x : (int)(blockIdx.x >> 1);       // CTA or CTA pair
  const int num_units = kCta == 1 ? (int)gridDim.x : (int)(gridDim.x >> 1);
  constexpr int kTileM = BM * kCta;
  const int num_m = (p.M + kTileM - 1) / kTileM;
  const int num_n = (p.N + BN - 1) / BN;
  const int tiles_per_group = num_m * num_n;
  const int num_tiles = p.group_mode == 2 ? tiles_per_group * p.num_groups : tiles_per_group;
  constexpr int kGroupM = kGroupRows / kTileM;
  // tile index -> (row tile, column tile): groups of kGroupM row tiles, row index fastest
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
  auto tile_info = [&](int t) {
    Tile ti;
    int tm, tn, e = 0;
    if (p.group_mode == 2) {
      e = t / tiles_per_group;
      t -= e * tiles_per_group;
    }
    tile_coord(t, tm, tn);
    if (kComm && p.m_rotate) tm = (tm + p.m_rotate) % num_m;
    ti.skip = 0;
    ti.m_base = tm * kTileM;
    ti.n0 = tn * BN;
    ti.c_row = ti.m_base;
    ti.b_row_off = 0;
    ti.k_beg = 0;
    ti.nkb = (p.K + BK - 1) / BK;
    if (p.group_mode == 1) {
      const int total = p.group_offs[p.num_groups];
      if (ti.m_base >= total) {
        ti.skip = 1;
      } else {
        int lo = 0, hi = p.num_groups;     // largest g with group_offs[g] <= m_base
        while (hi - lo > 1) {
          const int mid = (lo + hi) >> 1;
          if (p.group_offs[mid] <= ti.m_base) lo = mid; else hi = mid;
        }
        ti.b_row_off = lo * p.b_group_rows;
      }
    } else if (p.group_mode == 2) {
      ti.k_beg = p.group_offs[e];
      ti.nkb = (p.group_offs[e + 1] - ti.k_beg + BK - 1) / BK;
      ti.c_row = e * p.M + ti.m_base;
    }
    return ti;
  };

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(full_bar(s), kCta);      // one arrive.expect_tx per producing CTA
      mbar_init(empty_bar(s), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(tfull_bar(a), 1);
      mbar_init(tempty_bar(a), 4 * kCta);  // epilogue warps of every CTA of the pair
    }
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_b);
    tma_prefetch_desc(&tmap_c);
  }
  if (warp == 1) {
    // The whole TMEM of the SM: both CTAs of a pair therefore get base column 0.
    tmem_alloc(smem_u32(tmem_ptr_smem), kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  if constexpr (kCta == 2) cluster_sync();   // the peer's barriers exist before anyone signals them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_ptr_smem;

  if (warp == 0) {
    // ------------------------------------------------------------- TMA producer (every CTA)
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      for (int tile = unit; tile < num_tiles && ok; tile += num_units) {
        const Tile ti = tile_info(tile);
        if (ti.skip) continue;
        const int m0 = ti.m_base + (int)cta_rank * BM;
        const int n0 = ti.n0 + (int)cta_rank * C_::kBRows;
        if (kComm && p.a_flags != nullptr && m0 < p.M && m0 / p.gather_shard_rows != p.gather_rank) {
          // rows of another rank: wait (bounded) until the copy threads have brought this block in
          const uint32_t* f = p.a_flags + m0 / BM;
          const uint32_t epoch = *p.a_epoch;
          uint32_t seen = 0, spins = 0;
          while (true) {
            asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(seen) : "l"(f) : "memory");
            if ((int32_t)(seen - epoch) >= 0) break;
            if (++spins > kSpinLimit || *abort_flag) { *abort_flag = 1; ok = false; break; }
          }
          if (!ok) break;
          asm volatile("fence.proxy.async.global;" ::: "memory");   // the TMA engine reads what generic stores wrote
        }
        for (int kb = 0; kb < ti.nkb; ++kb, ++it) {
          const int s = it % kStages;
          const uint32_t parity = ((it / kStages) & 1u) ^ 1u;
          const bool got = kCta == 1 ? mbar_wait(empty_bar(s), parity, abort_flag)
                                     : mbar_wait_cluster(empty_bar(s), parity, abort_flag);
          if (!got) { ok = false; break; }
          const uint32_t sa = base + s * kStageBytes;
          const uint32_t sb = sa + kABytes;
          const int k0 = ti.k_beg + kb * BK;
          // bytes of both CTAs are counted by the barrier of CTA 0
          const uint32_t fb = kCta == 1 ? full_bar(s) : mapa(full_bar(s), 0);
          auto load = [&](uint32_t dst, const CUtensorMap* map, int c0, int c1) {
            if constexpr (kCta == 1) tma_load_2d(dst, map, fb, c0, c1);
            else tma_load_2d_pair(dst, map, fb, c0, c1);
          };
          auto load3 = [&](uint32_t dst, const CUtensorMap* map, int c1, int c2) {
            if constexpr (kCta == 1) tma_load_3d(dst, map, fb, 0, c1, c2);
            else tma_load_3d_pair(dst, map, fb, 0, c1, c2);
          };
          if (p.debug & 1) {
            if constexpr (kCta == 1) mbar_arrive(fb);
            else mbar_arrive_cluster(fb);
            continue;
          }
          if constexpr (kCta == 1) mbar_expect_tx(fb, kStageBytes);
          else mbar_expect_tx_cluster(fb, kStageBytes);
          if (!p.a_mn_major) {
            load(sa, &tmap_a, k0, m0);                                // box {64 k, 128 rows}
          } else if (p.a_mn3d) {
            load3(sa, &tmap_a, k0, m0 / 64);                          // box {64 m, 64 k-rows, BM / 64 blocks}
          } else {
#pragma unroll
            for (int b = 0; b < BM / 64; ++b)                         // boxes {64 m, 64 k-rows}
              load(sa + b * (BK * 128), &tmap_a, m0 + b * 64, k0);
          }
          if (!p.b_mn_major) {
            load(sb, &tmap_b, k0, n0 + ti.b_row_off);                 // box {64 k, kBRows rows}
          } else if (p.b_mn3d) {
            load3(sb, &tmap_b, k0 + ti.b_row_off, n0 / 64);
          } else {
#pragma unroll
            for (int b = 0; b < C_::kBRows / 64; ++b)
              load(sb + b * (BK * 128), &tmap_b, n0 + b * 64, k0 + ti.b_row_off);
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------- MMA issuer (CTA 0 of a pair)
    if (lane == 0 && cta_rank == 0) {
      const uint32_t idesc = make_idesc(p.a_mn_major != 0, p.b_mn_major != 0, kTileM, BN);
      // K-major: SBO = 1024 B between 8-row groups, one MMA K step = 32 B inside the swizzled row.
      // MN-major: LBO = BK*128 B between 64-column boxes, SBO = 1024 B between 8-k-row groups,
      //           one MMA K step = 16 k-rows = 2048 B.
      const uint32_t a_lbo = p.a_mn_major ? BK * 128 : 16, a_step = p.a_mn_major ? 2048 : 32;
      const uint32_t b_lbo = p.b_mn_major ? BK * 128 : 16, b_step = p.b_mn_major ? 2048 : 32;
      uint32_t it = 0, tcount = 0;
      bool ok = true;
      for (int tile = unit; tile < num_tiles && ok; tile += num_units) {
        const Tile ti = tile_info(tile);
        if (ti.skip) continue;
        const int num_kb = ti.nkb;
        const int acc = tcount & 1;
        const uint32_t acc_parity = ((tcount >> 1) & 1u) ^ 1u;
        ++tcount;
        const bool got = kCta == 1 ? mbar_wait(tempty_bar(acc), acc_parity, abort_flag)
                                   : mbar_wait_cluster(tempty_bar(acc), acc_parity, abort_flag);
        if (!got) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const int s = it % kStages;
          const uint32_t parity = (it / kStages) & 1u;
          const bool gotf = kCta == 1 ? mbar_wait(full_bar(s), parity, abort_flag)
                                      : mbar_wait_cluster(full_bar(s), parity, abort_flag);
          if (!gotf) { ok = false; break; }
          tc_fence_after();
          const uint32_t sa = base + s * kStageBytes;
          const uint32_t sb = sa + kABytes;
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            const uint64_t ad = make_desc(sa + k * a_step, a_lbo, 1024);
            const uint64_t bd = make_desc(sb + k * b_step, b_lbo, 1024);
            umma_bf16<kCta>(d_tmem, ad, bd, idesc, (kb | k) != 0 ? 1u : 0u);
          }
          // the stage can be refilled (in both CTAs) once these MMAs have read it
          if constexpr (kCta == 1) umma_commit(empty_bar(s));
          else umma_commit_pair(empty_bar(s), 3);
        }
        if (ok && num_kb > 0) {
          if constexpr (kCta == 1) umma_commit(tfull_bar(acc));
          else umma_commit_pair(tfull_bar(acc), 3);
        } else if (ok) {
          // an empty group: nothing was issued, the epilogue writes zeros
          mbar_arrive(tfull_bar(acc));
          if constexpr (kCta == 2) mbar_arrive_cluster(mapa(tfull_bar(acc), 1));
        }
      }
    }
  } else if (kComm && warp >= 6) {
    // ------------------------------------------------------------- shard copy threads (all-gather)
    if (p.gather_ranks > 1) {
      const int ct = (int)threadIdx.x - kThreads;
      const int per_shard = p.gather_shard_rows / BM;
      const int total = (p.gather_ranks - 1) * per_shard;
      const int n16 = BM * p.gather_row_bytes / 16;
      const uint32_t epoch = *p.a_epoch;
      for (int c = (int)blockIdx.x; c < total; c += (int)gridDim.x) {
        const int src = (p.gather_rank + 1 + c / per_shard) % p.gather_ranks;
        const int blk = src * per_shard + c % per_shard;
        const int64_t off = (int64_t)blk * BM * p.gather_row_bytes;
        const uint4* sp = reinterpret_cast<const uint4*>(p.gather_src[src] + off);
        uint4* dp = reinterpret_cast<uint4*>(p.gather_dst + off);
        for (int i = ct; i < n16; i += kCommThreads * 4) {
          uint4 v[4];
#pragma unroll
          for (int u = 0; u < 4; ++u)
            if (i + u * kCommThreads < n16) v[u] = sp[i + u * kCommThreads];
#pragma unroll
          for (int u = 0; u < 4; ++u)
            if (i + u * kCommThreads < n16) dp[i + u * kCommThreads] = v[u];
        }
        __threadfence();
        asm volatile("bar.sync 1, %0;" ::"n"(kCommThreads) : "memory");   // the four copy warps (no waits inside this loop)
        if (ct == 0) asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(p.a_flags + blk), "r"(epoch) : "memory");
      }
    }
  } else {
    // ------------------------------------------------------------- epilogue (warps 2..5, every CTA)
    const int q = warp & 3;  // TMEM lane quarter this warp may access
    uint32_t tcount = 0, sbuf = 0;
    bool ok = true;
    const uint32_t te_leader = kCta == 1 ? 0u : mapa(tempty_bar(0), 0);
    for (int tile = unit; tile < num_tiles && ok; tile += num_units) {
      const Tile ti = tile_info(tile);
      if (ti.skip) continue;
      const int acc = tcount & 1;
      const uint32_t acc_parity = (tcount >> 1) & 1u;
      ++tcount;
      const int m0 = ti.c_row + (int)cta_rank * BM;
      const int n0 = ti.n0;
      const bool got = kCta == 1 ? mbar_wait(tfull_bar(acc), acc_parity, abort_flag)
                                 : mbar_wait_cluster(tfull_bar(acc), acc_parity, abort_flag);
      if (!got) { ok = false; break; }
      tc_fence_after();
      {
        // 64 columns at a time go through a 128B-swizzled staging tile in shared memory and leave
        // as one TMA tile store, or a TMA reduce-add when accumulating into C (full 128-byte
        // lines; edges are clipped).
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
          if (lane == 0) tma_store_wait_read<1>();   // the tile written two steps ago has been read
          __syncwarp();
          const uint32_t buf = stage0 + (sbuf ? 4096u : 0u);
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            uint32_t w[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const int i = (j & 3) * 8 + 2 * e;
              const float lo = __uint_as_float(j < 4 ? r0[i] : r1[i]);
              const float hi = __uint_as_float(j < 4 ? r0[i + 1] : r1[i + 1]);
              __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
              w[e] = *reinterpret_cast<uint32_t*>(&h);
            }
            const uint32_t dst = buf + (uint32_t)lane * 128u + (uint32_t)((j ^ (lane & 7)) << 4);
            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(w[0]), "r"(w[1]), "r"(w[2]), "r"(w[3])
                         : "memory");
          }
          fence_proxy_async_smem();
          __syncwarp();
          const int col0 = n0 + c * 64;
          if (lane == 0 && col0 < p.N && m0 + q * 32 < p.c_rows && !(p.debug & 2)) {
            if (kComm && p.scatter_ranks > 0) {
              const int r0 = m0 + q * 32;
              const int dst = r0 / p.scatter_shard_rows;
              tma_store_2d(&cmaps.m[dst], buf, col0, p.scatter_rank * p.scatter_shard_rows + r0 % p.scatter_shard_rows);
            } else if (p.accumulate) {
              tma_reduce_add_2d(&tmap_c, buf, col0, m0 + q * 32);
            } else {
              tma_store_2d(&tmap_c, buf, col0, m0 + q * 32);
            }
            tma_store_commit();
          }
          sbuf ^= 1u;
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        if constexpr (kCta == 1) mbar_arrive(tempty_bar(acc));
        else mbar_arrive_cluster(te_leader + 8u * acc);
      }
    }
    if (lane == 0) {
      tma_store_wait<0>();   // shared memory must outlive the stores that read it
      if (kComm && p.scatter_ranks > 0) __threadfence_system();   // tiles stored into peers' staging buffers
    }
  }

  tc_fence_before();
  __syncthreads();
  // A CTA of a pair may not free its TMEM or leave while the other one can still issue MMAs
  // that read this CTA's shared memory and write its TMEM.
  if constexpr (kCta == 2) cluster_sync();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
  if (threadIdx.x == 0 && *abort_flag && p.status != nullptr) atomicOr(p.status, kStatusWaitTimedOut);
}

}  // namespace gemm

// ----------------------------------------------------------------------------------------
static CUtensorMap make_tmap_2d(const void* ptr, uint64_t inner, uint64_t outer, uint64_t row_stride_bytes,
                                uint32_t box_inner, uint32_t box_outer) {
  CUtensorMap map;
  const cuuint64_t dims[2] = {inner, outer};
  const cuuint64_t strides[1] = {row_stride_bytes};
  const cuuint32_t box[2] = {box_inner, box_outer};
  const cuuint32_t elem[2] = {1, 1};
  const CUresult r = cuTensorMapEncodeTiled(&map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims,
                                            strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                            CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  TORCH_CHECK(r == CUDA_SUCCESS, "cuTensorMapEncodeTiled failed with code ", (int)r);
  return map;
}

// MN-major operand [k_rows, mn] (row stride given) as [mn / 64][k_rows][64]: the box {64, BK, nblk} lands in shared memory
// as nblk consecutive 64-column boxes, the layout that nblk two-dimensional loads produce.  mn must be a multiple of 64.
static CUtensorMap make_tmap_mn3d(const void* ptr, uint64_t mn, uint64_t k_rows, uint64_t row_stride_bytes, uint32_t box_k,
                                  uint32_t nblk) {
  CUtensorMap map;
  const cuuint64_t dims[3] = {64, k_rows, mn / 64};
  const cuuint64_t strides[2] = {row_stride_bytes, 128};
  const cuuint32_t box[3] = {64, box_k, nblk};
  const cuuint32_t elem[3] = {1, 1, 1};
  const CUresult r = cuTensorMapEncodeTiled(&map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(ptr), dims,
                                            strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                            CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  TORCH_CHECK(r == CUDA_SUCCESS, "cuTensorMapEncodeTiled (3-D MN-major) failed with code ", (int)r);
  return map;
}

// MN-major operands whose extent divides by 64 use one 3-D load per stage instead of one 2-D load per 64-column box
// (2 to 4 per operand): measured 5-29 % faster on the weight- and input-gradient shapes of Llama-3 8B.  0 restores
// the 2-D boxes (timing comparisons).
static int g_gemm_mn3d = 1;
void gemm_set_mn3d(int64_t v) { g_gemm_mn3d = v != 0; }

static at::Tensor& gemm_status_tensor(const at::Device& dev) {
  static std::vector<at::Tensor> per_device(64);
  auto& t = per_device[dev.index()];
  if (!t.defined()) t = at::zeros({1}, at::TensorOptions().dtype(at::kInt).device(dev));
  return t;
}

static int g_gemm_debug = 0;
// Timing diagnostics that make the kernel skip part of its work (results are garbage by design).
// Refused unless the process was started with TB200_KERNEL_TIMING_DEBUG=1, so that no training
// job can switch them on by accident.
void gemm_set_debug(int64_t v) {
  TORCH_CHECK(v == 0 || std::getenv("TB200_KERNEL_TIMING_DEBUG") != nullptr,
              "gemm_set_debug: set TB200_KERNEL_TIMING_DEBUG=1 in the environment to enable the timing switches");
  g_gemm_debug = (int)v;
}
static int g_gemm_variant = 0;  // 0 = choose by shape, 1 = single CTA tiles, 2 = CTA-pair tiles

void gemm_set_variant(int64_t v) {
  TORCH_CHECK(v >= 0 && v <= 2, "gemm_set_variant: 0 (auto), 1 (single CTA) or 2 (CTA pair)");
  g_gemm_variant = (int)v;
}

template <int kCta, bool kComm = false>
static void launch_gemm(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tc_, const gemm::Params& p,
                        cudaStream_t stream, const gemm::CommMaps* comm_maps = nullptr) {
  using namespace gemm;
  using C_ = Cfg<kCta>;
  static bool attr_set = false;
  if (!attr_set) {
    C10_CUDA_CHECK(cudaFuncSetAttribute(gemm_bf16_kernel<kCta, kComm>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        C_::kSmemBytes));
    attr_set = true;
  }
  const int tile_m = BM * kCta;
  const int tiles = ((p.M + tile_m - 1) / tile_m) * ((p.N + BN - 1) / BN) * (p.group_mode == 2 ? p.num_groups : 1);
  cudaLaunchConfig_t cfg = {};
  cfg.blockDim = dim3(kThreads + (kComm ? kCommThreads : 0));
  cfg.dynamicSmemBytes = C_::kSmemBytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  if (kCta == 1) {
    cfg.gridDim = dim3(std::min(tiles, num_sms()));
    cfg.numAttrs = 0;
  } else {
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    // A persistent grid must be resident at once: ask how many CTA pairs the device can hold
    // (SM pairs that cannot host a cluster would otherwise serialise a second wave).
    static int max_pairs = 0;
    if (max_pairs == 0) {
      cfg.gridDim = dim3(num_sms() & ~1);
      int n = 0;
      C10_CUDA_CHECK(cudaOccupancyMaxActiveClusters(&n, gemm_bf16_kernel<kCta, kComm>, &cfg));
      max_pairs = std::max(1, std::min(n, num_sms() / 2));
    }
    cfg.gridDim = dim3(2 * std::min(tiles, max_pairs));
  }
  static const CommMaps no_maps = {};
  C10_CUDA_CHECK(cudaLaunchKernelEx(&cfg, gemm_bf16_kernel<kCta, kComm>, ta, tb, tc_, comm_maps ? *comm_maps : no_maps, p));
}

static void clear_comm(gemm::Params& p) {
  p.a_flags = nullptr; p.a_epoch = nullptr; p.m_rotate = 0;
  p.gather_ranks = 0; p.gather_rank = 0; p.gather_shard_rows = 1; p.gather_row_bytes = 0; p.gather_dst = nullptr;
  for (auto& g : p.gather_src) g = nullptr;
  p.scatter_ranks = 0; p.scatter_rank = 0; p.scatter_shard_rows = 1;
}

struct GroupArgs {
  const int* offs = nullptr;
  int num_groups = 0;
  int mode = 0;
  int b_group_rows = 0;
  int align = 0;        // every group offset is a multiple of this many rows
};

// Shared launcher.  a / b / c are the 2-D row-major views described by (rows, cols); the logical
// problem is M x N x K with A stored [K, M] when a_mn and B stored [K, N] when b_mn.
// lda / ldb / ldc: row strides in elements (negative: the operand is dense, stride = its column count).
static void run_gemm(const at::Tensor& ref, const void* a, int64_t a_rows, int64_t a_cols, const void* b, int64_t b_rows,
                     int64_t b_cols, void* c, int64_t c_rows, int64_t M, int64_t N, int64_t K, bool a_mn, bool b_mn,
                     bool accumulate, const GroupArgs& g, int64_t lda = -1, int64_t ldb = -1, int64_t ldc = -1) {
  using namespace gemm;
  c10::cuda::CUDAGuard guard(ref.device());
  // The tensor-map encoder is a driver-API call and needs the primary context current on this
  // thread; autograd worker threads may not have bound it yet.
  C10_CUDA_CHECK(cudaSetDevice(ref.device().index()));
  bool pair;
  if (g.mode == 1) pair = g.align % 256 == 0 && M >= 512;
  else if (g.mode == 2) pair = M % 256 == 0;
  else pair = M >= 512;   // the CTA pair pays off once a 256-row tile is full
  if (g_gemm_variant == 1 && !(g.mode == 2 && false)) pair = false;
  if (g_gemm_variant == 2 && (g.mode == 0 || (g.mode == 1 && g.align % 256 == 0) || (g.mode == 2 && M % 256 == 0))) pair = true;
  if (g.mode == 1) TORCH_CHECK(g.align % (pair ? 256 : 128) == 0, "grouped gemm: group offsets must be multiples of the row tile");
  if (g.mode == 2) TORCH_CHECK(M % (pair ? 256 : 128) == 0 && g.align % 64 == 0, "grouped gemm: M must be a multiple of the row tile");
  const uint32_t b_box_rows = pair ? Cfg<2>::kBRows : Cfg<1>::kBRows;
  // K-major: inner = K, box {64, rows};  MN-major: inner = MN extent, box {64, 64 k-rows}
  if (lda < 0) lda = a_cols;
  if (ldb < 0) ldb = b_cols;
  if (ldc < 0) ldc = N;
  const bool a3 = a_mn && g_gemm_mn3d && a_cols % 64 == 0, b3 = b_mn && g_gemm_mn3d && b_cols % 64 == 0;
  const CUtensorMap ta = a3 ? make_tmap_mn3d(a, a_cols, a_rows, lda * 2, BK, BM / 64)
                         : a_mn ? make_tmap_2d(a, a_cols, a_rows, lda * 2, 64, BK)
                                : make_tmap_2d(a, a_cols, a_rows, lda * 2, BK, BM);
  const CUtensorMap tb = b3 ? make_tmap_mn3d(b, b_cols, b_rows, ldb * 2, BK, b_box_rows / 64)
                         : b_mn ? make_tmap_2d(b, b_cols, b_rows, ldb * 2, 64, BK)
                                : make_tmap_2d(b, b_cols, b_rows, ldb * 2, BK, b_box_rows);
  const CUtensorMap tcm = make_tmap_2d(c, N, c_rows, ldc * 2, 64, 32);   // store tiles: 64 columns x 32 rows
  Params p;
  p.M = (int)M; p.N = (int)N; p.K = (int)K;
  p.a_mn_major = a_mn; p.b_mn_major = b_mn; p.accumulate = accumulate ? 1 : 0;
  p.a_mn3d = a3; p.b_mn3d = b3;
  p.debug = g_gemm_debug;
  p.C = reinterpret_cast<__nv_bfloat16*>(c);
  p.status = gemm_status_tensor(ref.device()).data_ptr<int>();
  p.group_offs = g.offs; p.num_groups = g.num_groups; p.group_mode = g.mode; p.b_group_rows = g.b_group_rows;
  p.c_rows = (int)c_rows;
  clear_comm(p);
  auto stream = at::cuda::getCurrentCUDAStream();
  if (pair) launch_gemm<2>(ta, tb, tcm, p, stream);
  else launch_gemm<1>(ta, tb, tcm, p, stream);
}

static void check_bf16_2d(const at::Tensor& t, const char* name) {
  TORCH_CHECK(t.is_cuda() && t.scalar_type() == at::kBFloat16 && t.is_contiguous(), "gemm: ", name,
              " must be a contiguous CUDA bf16 tensor");
  TORCH_CHECK((reinterpret_cast<uintptr_t>(t.data_ptr()) & 15) == 0, "gemm: ", name, " must be 16-byte aligned");
}

// mode: 0 = NT (a[M,K], b[N,K]), 1 = NN (a[M,K], b[K,N]), 2 = TN (a[K,M], b[K,N]).
void gemm_bf16(const at::Tensor& a, const at::Tensor& b, at::Tensor c, int64_t mode, bool accumulate) {
  check_bf16_2d(a, "a"); check_bf16_2d(b, "b"); check_bf16_2d(c, "c");
  TORCH_CHECK(a.dim() == 2 && b.dim() == 2 && c.dim() == 2);
  const bool a_mn = mode == 2, b_mn = mode != 0;
  const int64_t M = a_mn ? a.size(1) : a.size(0);
  const int64_t K = a_mn ? a.size(0) : a.size(1);
  const int64_t N = b_mn ? b.size(1) : b.size(0);
  TORCH_CHECK((b_mn ? b.size(0) : b.size(1)) == K, "gemm_bf16: inner dimensions differ");
  TORCH_CHECK(c.size(0) == M && c.size(1) == N, "gemm_bf16: bad output shape");
  // Row strides of every operand must be multiples of 16 bytes (TMA).
  TORCH_CHECK(N % 8 == 0, "gemm_bf16: N must be a multiple of 8");
  TORCH_CHECK(a_mn ? (M % 8 == 0) : (K % 8 == 0), "gemm_bf16: the contiguous dimension of A must be a multiple of 8");
  TORCH_CHECK(b_mn || K % 8 == 0, "gemm_bf16: the contiguous dimension of B must be a multiple of 8");
  if (M == 0 || N == 0) return;
  run_gemm(a, a.data_ptr(), a.size(0), a.size(1), b.data_ptr(), b.size(0), b.size(1), c.data_ptr(), M, M, N, K, a_mn, b_mn,
           accumulate, GroupArgs());
}

// Grouped GEMM over rows sorted by group (tokens sorted by expert).  offs: int32 [G + 1] on the
// device, offs[g] = first row of group g, offs[G] = number of valid rows, all multiples of `align`
// (128 or 256): groups are padded, padded rows of the inputs are zero.
//   mode 0: c[rows of g] = a[rows of g] . b[g]^T      a [R, K], b [G, N, K], c [R, N]
//   mode 1: c[rows of g] = a[rows of g] . b[g]        a [R, K], b [G, K, N], c [R, N]
//   mode 2: c[g] = a[rows of g]^T . b[rows of g]      a [R, M], b [R, N],    c [G, M, N]
// Rows of c at or beyond offs[G] (modes 0, 1) are not written.
// A row-major 2-D operand whose rows may be strided (a column slice of a wider buffer): unit column stride, row
// stride and base address multiples of 16 bytes (the tensor-map rules).
static void check_bf16_rows(const at::Tensor& t, const char* name) {
  TORCH_CHECK(t.is_cuda() && t.scalar_type() == at::kBFloat16 && t.dim() == 2 && (t.size(1) == 1 || t.stride(1) == 1) &&
                  t.stride(0) >= t.size(1) && (t.stride(0) * 2) % 16 == 0,
              "gemm: ", name, " must be a 2-D CUDA bf16 tensor with contiguous rows and a 16-byte multiple row stride");
  TORCH_CHECK((reinterpret_cast<uintptr_t>(t.data_ptr()) & 15) == 0, "gemm: ", name, " must be 16-byte aligned");
}

void gemm_grouped_bf16(const at::Tensor& a, const at::Tensor& b, at::Tensor c, const at::Tensor& offs, int64_t mode,
                       int64_t align, bool accumulate) {
  // the row-indexed operands (a, and c in modes 0 / 1, b in mode 2) may be column slices of wider buffers
  check_bf16_rows(a, "a");
  if (mode == 2) { check_bf16_rows(b, "b"); check_bf16_2d(c, "c"); }
  else { check_bf16_2d(b, "b"); check_bf16_rows(c, "c"); }
  TORCH_CHECK(offs.is_cuda() && offs.scalar_type() == at::kInt && offs.is_contiguous() && offs.numel() >= 2,
              "gemm_grouped_bf16: offs must be an int32 CUDA tensor of G + 1 entries");
  const int G = (int)offs.numel() - 1;
  GroupArgs g;
  g.offs = offs.data_ptr<int>();
  g.num_groups = G;
  g.align = (int)align;
  TORCH_CHECK(a.dim() == 2, "gemm_grouped_bf16: a must be 2-D");
  const int64_t R = a.size(0);
  if (R == 0) return;
  if (mode == 0 || mode == 1) {
    TORCH_CHECK(b.dim() == 3 && b.size(0) == G && c.dim() == 2 && c.size(0) == R);
    const int64_t K = a.size(1);
    const int64_t N = mode == 0 ? b.size(1) : b.size(2);
    TORCH_CHECK((mode == 0 ? b.size(2) : b.size(1)) == K && c.size(1) == N, "gemm_grouped_bf16: shapes do not match");
    TORCH_CHECK(K % 8 == 0 && N % 8 == 0);
    if (mode == 1) TORCH_CHECK(K % 64 == 0, "gemm_grouped_bf16: mode 1 needs K to be a multiple of 64");
    g.mode = 1;
    g.b_group_rows = (int)(mode == 0 ? N : K);
    run_gemm(a, a.data_ptr(), R, K, b.data_ptr(), (int64_t)G * b.size(1), b.size(2), c.data_ptr(), R, R, N, K, false,
             mode == 1, accumulate, g, a.stride(0), -1, c.stride(0));
  } else {
    TORCH_CHECK(mode == 2 && b.dim() == 2 && b.size(0) == R && c.dim() == 3 && c.size(0) == G);
    const int64_t M = a.size(1), N = b.size(1);
    TORCH_CHECK(c.size(1) == M && c.size(2) == N && M % 8 == 0 && N % 8 == 0);
    g.mode = 2;
    run_gemm(a, a.data_ptr(), R, M, b.data_ptr(), R, N, c.data_ptr(), (int64_t)G * M, M, N, R, true, true, accumulate, g,
             a.stride(0), b.stride(0), -1);
  }
}

// ---- tensor-parallel GEMMs with the collective inside the kernel --------------------------
// All-gather -> GEMM.  `a_gather` is this rank's gather buffer [ranks * shard_rows, K] in symmetric
// memory with the rank's own rows already in place; `peer_ptrs[r]` is the address of rank r's
// gather buffer; `flags` (uint32 [ranks * shard_rows / 128], zero-initialised once) and the
// monotonically increasing `epoch` (a one-element int32 device tensor that the caller increments in
// stream order before each call, e.g. through the `bump` argument of symm_barrier) tell the GEMM
// which row blocks have arrived.  Every rank must have passed a barrier after writing its own rows
// and before this call.
//   mode 0: c = gathered . b^T (b [N, K]);  mode 1: c = gathered . b (b [K, N]).
void gemm_allgather_bf16(const at::Tensor& a_gather, const at::Tensor& b, at::Tensor c, at::IntArrayRef peer_ptrs,
                         int64_t rank, at::Tensor flags, const at::Tensor& epoch, int64_t mode) {
  using namespace gemm;
  check_bf16_2d(a_gather, "a_gather"); check_bf16_2d(b, "b"); check_bf16_2d(c, "c");
  TORCH_CHECK(mode == 0 || mode == 1, "gemm_allgather_bf16: mode 0 (NT) or 1 (NN)");
  const int R = (int)peer_ptrs.size();
  TORCH_CHECK(R >= 1 && R <= 8 && rank >= 0 && rank < R, "gemm_allgather_bf16: 1..8 ranks");
  const int64_t M = a_gather.size(0), K = a_gather.size(1);
  const int64_t N = mode == 0 ? b.size(0) : b.size(1);
  TORCH_CHECK((mode == 0 ? b.size(1) : b.size(0)) == K && c.size(0) == M && c.size(1) == N);
  TORCH_CHECK(M % R == 0 && (M / R) % 256 == 0, "gemm_allgather_bf16: the shard must be a multiple of 256 rows");
  TORCH_CHECK(K % 8 == 0 && N % 8 == 0);
  TORCH_CHECK(flags.is_cuda() && flags.scalar_type() == at::kInt && flags.numel() >= M / BM && flags.is_contiguous());
  TORCH_CHECK(epoch.is_cuda() && epoch.scalar_type() == at::kInt && epoch.numel() == 1, "gemm_allgather_bf16: epoch is an int32[1] device tensor");
  c10::cuda::CUDAGuard guard(a_gather.device());
  C10_CUDA_CHECK(cudaSetDevice(a_gather.device().index()));
  const bool b_mn = mode == 1;
  const CUtensorMap ta = make_tmap_2d(a_gather.data_ptr(), K, M, K * 2, BK, BM);
  const CUtensorMap tb = b_mn ? make_tmap_2d(b.data_ptr(), N, K, N * 2, 64, BK)
                              : make_tmap_2d(b.data_ptr(), K, N, K * 2, BK, Cfg<2>::kBRows);
  const CUtensorMap tcm = make_tmap_2d(c.data_ptr(), N, M, N * 2, 64, 32);
  Params p;
  p.M = (int)M; p.N = (int)N; p.K = (int)K;
  p.a_mn_major = 0; p.b_mn_major = b_mn; p.accumulate = 0; p.debug = 0;
  p.a_mn3d = 0; p.b_mn3d = 0;
  p.C = reinterpret_cast<__nv_bfloat16*>(c.data_ptr());
  p.status = gemm_status_tensor(a_gather.device()).data_ptr<int>();
  p.group_offs = nullptr; p.num_groups = 0; p.group_mode = 0; p.b_group_rows = 0; p.c_rows = (int)M;
  clear_comm(p);
  const int shard = (int)(M / R);
  p.a_flags = reinterpret_cast<uint32_t*>(flags.data_ptr<int>());
  p.a_epoch = reinterpret_cast<const uint32_t*>(epoch.data_ptr<int>());
  p.m_rotate = (int)rank * (shard / (2 * BM));
  p.gather_ranks = R; p.gather_rank = (int)rank; p.gather_shard_rows = shard; p.gather_row_bytes = (int)(K * 2);
  for (int r = 0; r < R; ++r) p.gather_src[r] = reinterpret_cast<const uint8_t*>(static_cast<uintptr_t>(peer_ptrs[r]));
  p.gather_dst = reinterpret_cast<uint8_t*>(a_gather.data_ptr());
  launch_gemm<2, true>(ta, tb, tcm, p, at::cuda::getCurrentCUDAStream());
}

// GEMM -> reduce-scatter, first half: every tile of this rank's partial product [M, N] is stored
// into the staging buffer [ranks, M / ranks, N] of the rank that owns its rows, in slot `rank`
// (TMA stores to peer memory from the epilogue).  After a barrier, `sum_slots` of the local staging
// buffer gives this rank's rows of the sum.  mode 0: a . b^T, mode 1: a . b.
void gemm_scatter_bf16(const at::Tensor& a, const at::Tensor& b, at::IntArrayRef staging_ptrs, int64_t rank, int64_t mode) {
  using namespace gemm;
  check_bf16_2d(a, "a"); check_bf16_2d(b, "b");
  TORCH_CHECK(mode == 0 || mode == 1);
  const int R = (int)staging_ptrs.size();
  TORCH_CHECK(R >= 1 && R <= 8 && rank >= 0 && rank < R);
  const int64_t M = a.size(0), K = a.size(1);
  const int64_t N = mode == 0 ? b.size(0) : b.size(1);
  TORCH_CHECK((mode == 0 ? b.size(1) : b.size(0)) == K);
  TORCH_CHECK(M % R == 0 && (M / R) % 256 == 0, "gemm_scatter_bf16: the shard must be a multiple of 256 rows");
  TORCH_CHECK(K % 8 == 0 && N % 8 == 0);
  c10::cuda::CUDAGuard guard(a.device());
  C10_CUDA_CHECK(cudaSetDevice(a.device().index()));
  const bool b_mn = mode == 1;
  const CUtensorMap ta = make_tmap_2d(a.data_ptr(), K, M, K * 2, BK, BM);
  const CUtensorMap tb = b_mn ? make_tmap_2d(b.data_ptr(), N, K, N * 2, 64, BK)
                              : make_tmap_2d(b.data_ptr(), K, N, K * 2, BK, Cfg<2>::kBRows);
  CommMaps maps = {};
  for (int r = 0; r < R; ++r)
    maps.m[r] = make_tmap_2d(reinterpret_cast<const void*>(static_cast<uintptr_t>(staging_ptrs[r])), N, M, N * 2, 64, 32);
  Params p;
  p.M = (int)M; p.N = (int)N; p.K = (int)K;
  p.a_mn_major = 0; p.b_mn_major = b_mn; p.accumulate = 0; p.debug = 0;
  p.a_mn3d = 0; p.b_mn3d = 0;
  p.C = nullptr;
  p.status = gemm_status_tensor(a.device()).data_ptr<int>();
  p.group_offs = nullptr; p.num_groups = 0; p.group_mode = 0; p.b_group_rows = 0; p.c_rows = (int)M;
  clear_comm(p);
  const int shard = (int)(M / R);
  p.scatter_ranks = R; p.scatter_rank = (int)rank; p.scatter_shard_rows = shard;
  p.m_rotate = (int)((rank + 1) % R) * (shard / (2 * BM));
  launch_gemm<2, true>(ta, tb, maps.m[rank], p, at::cuda::getCurrentCUDAStream(), &maps);
}

// out[rows, N] = sum over slots of staging[slot, rows, N] (fp32 accumulation).
__global__ void sum_slots_kernel(const __nv_bfloat16* __restrict__ st, __nv_bfloat16* __restrict__ out, int64_t n_vec,
                                 int slots) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n_vec) return;
  float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  for (int s = 0; s < slots; ++s) {
    float v[8];
    unpack8(reinterpret_cast<const bf16x8*>(st)[(int64_t)s * n_vec + i], v);
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] += v[j];
  }
  reinterpret_cast<bf16x8*>(out)[i] = pack8(acc);
}

at::Tensor sum_slots(const at::Tensor& staging) {
  TORCH_CHECK(staging.is_cuda() && staging.scalar_type() == at::kBFloat16 && staging.dim() == 3 && staging.is_contiguous());
  TORCH_CHECK((staging.size(1) * staging.size(2)) % 8 == 0);
  c10::cuda::CUDAGuard guard(staging.device());
  auto out = at::empty({staging.size(1), staging.size(2)}, staging.options());
  const int64_t n_vec = out.numel() / 8;
  if (n_vec > 0)
    sum_slots_kernel<<<(unsigned)((n_vec + 255) / 256), 256, 0, at::cuda::getCurrentCUDAStream()>>>(
        reinterpret_cast<const __nv_bfloat16*>(staging.data_ptr()), reinterpret_cast<__nv_bfloat16*>(out.data_ptr()), n_vec,
        (int)staging.size(0));
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  return out;
}

int64_t gemm_status(bool clear) {
  int dev = 0;
  cudaGetDevice(&dev);
  auto& t = gemm_status_tensor(at::Device(at::kCUDA, dev));
  const int64_t v = t.item<int>();
  if (clear && v) t.zero_();
  return v;
}

}  // namespace tb200
