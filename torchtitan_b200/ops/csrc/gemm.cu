// bf16 GEMM on the 5th-generation tensor cores: tcgen05.mma with TMEM accumulators,
// operands staged by TMA into 128B-swizzled shared memory, persistent warp-specialised CTAs.
//
//   mode 0 (NT): C[M,N] = A[M,K] . B[N,K]^T      forward of a linear layer
//   mode 1 (NN): C[M,N] = A[M,K] . B[K,N]        input gradient
//   mode 2 (TN): C[M,N] = A[K,M]^T . B[K,N]      weight gradient
// `accumulate` adds the product to the existing C (bf16) in the epilogue.
//
// One CTA per SM, tile 128 x 256, K step 64, 4-stage TMA pipeline (48 KB per stage).
//   warp 0      : TMA producer (one elected lane)
//   warp 1      : allocates TMEM, issues tcgen05.mma (one elected lane), commits to mbarriers
//   warps 2..5  : epilogue; each warp owns the 32 TMEM lanes of its quarter (warp_id % 4),
//                 reads the fp32 accumulator with tcgen05.ld, converts and stores bf16
// The 512 TMEM columns hold two 128 x 256 fp32 accumulators, so the epilogue of tile i
// overlaps the main loop of tile i+1.
//
// Operand layouts.  K-major operands ([rows, K] row-major) are loaded as boxes of 64 K-elements
// (128 B) x rows; MN-major operands ([K, cols] row-major) as boxes of 64 columns (128 B) x 64
// K-rows, one box per 64 columns.  Both use the 128-byte swizzle, which is what the shared
// memory matrix descriptors below describe.
//
// Every mbarrier wait is bounded: after kSpinLimit polls the waiter raises an abort flag in
// shared memory, all roles leave their loops, TMEM is freed and the kernel sets bit
// kStatusWaitTimedOut in the status word.  TMA loads are plain (no cluster multicast).
#include <ATen/ATen.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <cuda.h>

#include "common.cuh"

namespace tb200 {

namespace gemm {

constexpr int BM = 128;
constexpr int BN = 256;
constexpr int BK = 64;
constexpr int kStages = 4;
constexpr int UMMA_K = 16;
constexpr int kThreads = 192;
constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kABytes = BM * BK * 2;   // 16 KB
constexpr uint32_t kBBytes = BN * BK * 2;   // 32 KB
constexpr uint32_t kStageBytes = kABytes + kBBytes;
constexpr uint32_t kSmemBytes = kStages * kStageBytes + 1024 /*alignment slack*/ + 256 /*barriers*/;
constexpr uint32_t kSpinLimit = 20u * 1000u * 1000u;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait: false when the limit was hit or another role already aborted.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
  for (uint32_t i = 0; i < kSpinLimit; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((i & 1023u) == 1023u && *abort_flag) return false;
  }
  *abort_flag = 1;
  return false;
}

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1)
      : "memory");
}

__device__ __forceinline__ void tmem_alloc(uint32_t dst_smem, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                          uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Arrive on an mbarrier once all previously issued tcgen05.mma of this thread have completed.
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor (sm_100 format, 128-byte swizzle).
//   bits [0,14)  start address >> 4      bits [16,30) leading byte offset >> 4
//   bits [32,46) stride byte offset >> 4 bits [46,48) version = 1      bits [61,64) layout = 2 (SW128)
__device__ __forceinline__ uint64_t make_desc(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr & 0x3FFFFu) >> 4);
  d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFFu) << 16;
  d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFFu) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}

// Instruction descriptor for kind::f16: D fp32, A/B bf16, majorness per operand, N and M.
__host__ __device__ constexpr uint32_t make_idesc(bool a_mn_major, bool b_mn_major) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((a_mn_major ? 1u : 0u) << 15) | ((b_mn_major ? 1u : 0u) << 16) |
         ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
}

struct Params {
  int M, N, K;
  int a_mn_major;  // A is stored [K, M]
  int b_mn_major;  // B is stored [K, N]
  int accumulate;
  __nv_bfloat16* C;
  int* status;
};

__global__ void __launch_bounds__(kThreads, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                 const Params p) {
  extern __shared__ uint8_t smem_raw[];
  // stage buffers need 1024-byte alignment for the 128B swizzle atoms
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* gen_base = smem_raw + (base - raw);
  const uint32_t bar_base = base + kStages * kStageBytes;
  // barrier layout: full[kStages], empty[kStages], tmem_full[2], tmem_empty[2], then tmem ptr, abort flag
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (kStages + s); };
  auto tfull_bar = [&](int a) { return bar_base + 8u * (2 * kStages + a); };
  auto tempty_bar = [&](int a) { return bar_base + 8u * (2 * kStages + 2 + a); };
  uint32_t* tmem_ptr_smem = reinterpret_cast<uint32_t*>(gen_base + kStages * kStageBytes + 8 * (2 * kStages + 4));
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_ptr_smem + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int num_m = (p.M + BM - 1) / BM;
  const int num_n = (p.N + BN - 1) / BN;
  const int num_tiles = num_m * num_n;
  const int num_kb = (p.K + BK - 1) / BK;

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
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&tmap_a) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&tmap_b) : "memory");
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_ptr_smem), kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_ptr_smem;

  if (warp == 0) {
    // ------------------------------------------------------------- TMA producer
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        const int m0 = (tile % num_m) * BM;
        const int n0 = (tile / num_m) * BN;
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const int s = it % kStages;
          const uint32_t parity = ((it / kStages) & 1u) ^ 1u;
          if (!mbar_wait(empty_bar(s), parity, abort_flag)) { ok = false; break; }
          const uint32_t sa = base + s * kStageBytes;
          const uint32_t sb = sa + kABytes;
          mbar_expect_tx(full_bar(s), kStageBytes);
          const int k0 = kb * BK;
          if (!p.a_mn_major) {
            tma_load_2d(sa, &tmap_a, full_bar(s), k0, m0);            // box {64 k, 128 rows}
          } else {
#pragma unroll
            for (int b = 0; b < BM / 64; ++b)                         // boxes {64 m, 64 k-rows}
              tma_load_2d(sa + b * (BK * 128), &tmap_a, full_bar(s), m0 + b * 64, k0);
          }
          if (!p.b_mn_major) {
            tma_load_2d(sb, &tmap_b, full_bar(s), k0, n0);            // box {64 k, 256 rows}
          } else {
#pragma unroll
            for (int b = 0; b < BN / 64; ++b)
              tma_load_2d(sb + b * (BK * 128), &tmap_b, full_bar(s), n0 + b * 64, k0);
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      const uint32_t idesc = make_idesc(p.a_mn_major != 0, p.b_mn_major != 0);
      // K-major: SBO = 1024 B between 8-row groups, one MMA K step = 32 B inside the swizzled row.
      // MN-major: LBO = BK*128 B between 64-column boxes, SBO = 1024 B between 8-k-row groups,
      //           one MMA K step = 16 k-rows = 2048 B.
      const uint32_t a_lbo = p.a_mn_major ? BK * 128 : 16, a_step = p.a_mn_major ? 2048 : 32;
      const uint32_t b_lbo = p.b_mn_major ? BK * 128 : 16, b_step = p.b_mn_major ? 2048 : 32;
      uint32_t it = 0, tcount = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++tcount) {
        const int acc = tcount & 1;
        const uint32_t acc_parity = ((tcount >> 1) & 1u) ^ 1u;
        if (!mbar_wait(tempty_bar(acc), acc_parity, abort_flag)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const int s = it % kStages;
          const uint32_t parity = (it / kStages) & 1u;
          if (!mbar_wait(full_bar(s), parity, abort_flag)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sa = base + s * kStageBytes;
          const uint32_t sb = sa + kABytes;
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            const uint64_t ad = make_desc(sa + k * a_step, a_lbo, 1024);
            const uint64_t bd = make_desc(sb + k * b_step, b_lbo, 1024);
            umma_bf16(d_tmem, ad, bd, idesc, (kb | k) != 0 ? 1u : 0u);
          }
          umma_commit(empty_bar(s));  // the stage can be refilled once these MMAs have read it
        }
        if (ok) umma_commit(tfull_bar(acc));
      }
    }
  } else {
    // ------------------------------------------------------------- epilogue (warps 2..5)
    const int q = warp & 3;  // TMEM lane quarter this warp may access
    uint32_t tcount = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++tcount) {
      const int acc = tcount & 1;
      const uint32_t acc_parity = (tcount >> 1) & 1u;
      const int m0 = (tile % num_m) * BM;
      const int n0 = (tile / num_m) * BN;
      if (!mbar_wait(tfull_bar(acc), acc_parity, abort_flag)) { ok = false; break; }
      tc_fence_after();
      const int row = m0 + q * 32 + lane;
      __nv_bfloat16* crow = p.C + (int64_t)row * p.N;
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(acc * BN + c * 32);
        tmem_ld32(taddr, r);
        tmem_ld_wait();
        const int col0 = n0 + c * 32;
        if (row < p.M && col0 < p.N) {
          if (col0 + 32 <= p.N) {
#pragma unroll
            for (int v = 0; v < 4; ++v) {
              float f[8];
#pragma unroll
              for (int j = 0; j < 8; ++j) f[j] = __uint_as_float(r[v * 8 + j]);
              bf16x8* dst = reinterpret_cast<bf16x8*>(crow + col0 + v * 8);
              if (p.accumulate) {
                float o[8];
                unpack8(*dst, o);
#pragma unroll
                for (int j = 0; j < 8; ++j) f[j] += o[j];
              }
              *dst = pack8(f);
            }
          } else {
            for (int j = 0; j < 32 && col0 + j < p.N; ++j) {
              float f = __uint_as_float(r[j]);
              if (p.accumulate) f += __bfloat162float(crow[col0 + j]);
              crow[col0 + j] = __float2bfloat16_rn(f);
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(tempty_bar(acc));
    }
  }

  tc_fence_before();
  __syncthreads();
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

static at::Tensor& gemm_status_tensor(const at::Device& dev) {
  static std::vector<at::Tensor> per_device(64);
  auto& t = per_device[dev.index()];
  if (!t.defined()) t = at::zeros({1}, at::TensorOptions().dtype(at::kInt).device(dev));
  return t;
}

// mode: 0 = NT (a[M,K], b[N,K]), 1 = NN (a[M,K], b[K,N]), 2 = TN (a[K,M], b[K,N]).
void gemm_bf16(const at::Tensor& a, const at::Tensor& b, at::Tensor c, int64_t mode, bool accumulate) {
  TORCH_CHECK(a.is_cuda() && b.is_cuda() && c.is_cuda());
  TORCH_CHECK(a.scalar_type() == at::kBFloat16 && b.scalar_type() == at::kBFloat16 && c.scalar_type() == at::kBFloat16);
  TORCH_CHECK(a.dim() == 2 && b.dim() == 2 && c.dim() == 2 && a.is_contiguous() && b.is_contiguous() && c.is_contiguous());
  const bool a_mn = mode == 2, b_mn = mode != 0;
  const int64_t M = a_mn ? a.size(1) : a.size(0);
  const int64_t K = a_mn ? a.size(0) : a.size(1);
  const int64_t N = b_mn ? b.size(1) : b.size(0);
  TORCH_CHECK((b_mn ? b.size(0) : b.size(1)) == K, "gemm_bf16: inner dimensions differ");
  TORCH_CHECK(c.size(0) == M && c.size(1) == N, "gemm_bf16: bad output shape");
  // Row strides of every operand must be multiples of 16 bytes (TMA), and the epilogue stores 16-byte vectors.
  TORCH_CHECK(N % 8 == 0, "gemm_bf16: N must be a multiple of 8");
  TORCH_CHECK(a_mn ? (M % 8 == 0) : (K % 8 == 0), "gemm_bf16: the contiguous dimension of A must be a multiple of 8");
  TORCH_CHECK(b_mn || K % 8 == 0, "gemm_bf16: the contiguous dimension of B must be a multiple of 8");
  TORCH_CHECK((reinterpret_cast<uintptr_t>(a.data_ptr()) & 15) == 0 && (reinterpret_cast<uintptr_t>(b.data_ptr()) & 15) == 0 &&
              (reinterpret_cast<uintptr_t>(c.data_ptr()) & 15) == 0, "gemm_bf16: operands must be 16-byte aligned");
  if (M == 0 || N == 0) return;
  c10::cuda::CUDAGuard guard(a.device());
  // The tensor-map encoder is a driver-API call and needs the primary context current on this
  // thread; autograd worker threads may not have bound it yet.
  C10_CUDA_CHECK(cudaSetDevice(a.device().index()));
  using namespace gemm;
  // K-major: inner = K, box {64, rows};  MN-major: inner = MN extent, box {64, 64 k-rows}
  const CUtensorMap ta = a_mn ? make_tmap_2d(a.data_ptr(), M, K, M * 2, 64, BK)
                              : make_tmap_2d(a.data_ptr(), K, M, K * 2, BK, BM);
  const CUtensorMap tb = b_mn ? make_tmap_2d(b.data_ptr(), N, K, N * 2, 64, BK)
                              : make_tmap_2d(b.data_ptr(), K, N, K * 2, BK, BN);
  Params p;
  p.M = (int)M; p.N = (int)N; p.K = (int)K;
  p.a_mn_major = a_mn; p.b_mn_major = b_mn; p.accumulate = accumulate ? 1 : 0;
  p.C = reinterpret_cast<__nv_bfloat16*>(c.data_ptr());
  p.status = gemm_status_tensor(a.device()).data_ptr<int>();
  static bool attr_set = false;
  if (!attr_set) {
    C10_CUDA_CHECK(cudaFuncSetAttribute(gemm_bf16_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes));
    attr_set = true;
  }
  const int tiles = (int)(((M + BM - 1) / BM) * ((N + BN - 1) / BN));
  const int grid = std::min(tiles, num_sms());
  auto stream = at::cuda::getCurrentCUDAStream();
  gemm_bf16_kernel<<<grid, kThreads, kSmemBytes, stream>>>(ta, tb, p);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
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
