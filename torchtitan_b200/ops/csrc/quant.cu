// Block-scaled fp8 quantisation kernels.
//
// MXFP8 (OCP microscaling): blocks of 32 elements along the contraction dimension share one
// e8m0 (power-of-two) scale, the elements are e4m3.  The scale exponent is rounded up
// ("RCEIL": 2^e >= amax / 448), so no element saturates.  `axis = 1` scales along the last
// (contiguous) dimension, `axis = 0` along the first; the data keeps the input's [R, C] layout
// either way, the scales are [R, C/32] or [R/32, C].
//   mxfp8_quantize      bf16 -> (e4m3 bytes, e8m0 bytes)
//   mxfp8_dequantize    (e4m3, e8m0) -> bf16
//   mxfp8_fake_quant    bf16 -> bf16 holding exactly the values the MXFP8 pair represents
//                       (one pass; used by the linear layers' emulated GEMM path)
// Float8 row-wise: one fp32 scale per row, e4m3 data (float8_rowwise_quantize / fake_quant).
#include <ATen/ATen.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <cuda_fp8.h>

#include "common.cuh"

namespace tb200 {

constexpr float kE4M3Max = 448.f;

// e8m0 exponent byte of the smallest power of two >= amax / 448 (0 for an all-zero block).
__device__ __forceinline__ uint32_t e8m0_rceil(float amax) {
  if (!(amax > 0.f)) return 0u;
  const uint32_t bits = __float_as_uint(__fdiv_rn(amax, kE4M3Max));
  uint32_t e = (bits >> 23) & 0xffu;
  if (bits & 0x7fffffu) e += 1;            // round the exponent up
  return min(max(e, 1u), 254u);
}
__device__ __forceinline__ float e8m0_to_float(uint32_t e) { return __uint_as_float(e << 23); }        // 2^(e-127)
__device__ __forceinline__ float e8m0_inverse(uint32_t e) { return __uint_as_float((254u - e) << 23); } // 2^(127-e)

__device__ __forceinline__ uint32_t to_e4m3x4(float a, float b, float c, float d) {
  const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(a, b), __NV_SATFINITE, __NV_E4M3);
  const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(c, d), __NV_SATFINITE, __NV_E4M3);
  return lo | (hi << 16);
}
__device__ __forceinline__ float from_e4m3(uint32_t byte) {
  const __half_raw h = __nv_cvt_fp8_to_halfraw((__nv_fp8_storage_t)byte, __NV_E4M3);
  return __half2float(*reinterpret_cast<const __half*>(&h));
}

// ---- axis 1: 4 consecutive lanes own one block of 32 contiguous elements (8 each)
// kTiled: scales go to the 512-byte atoms (128 rows x 4 blocks) that the block-scaled MMA reads
// through tcgen05.cp: byte (r % 32) * 16 + (r / 32) * 4 + b inside atom (row tile, k tile).
template <bool kFake, bool kTiled = false>
__global__ void mx_rowwise_kernel(const __nv_bfloat16* __restrict__ x, uint8_t* __restrict__ data,
                                  uint8_t* __restrict__ scales, __nv_bfloat16* __restrict__ fake, int64_t n_vec, int C,
                                  const uint8_t* __restrict__ row_exp = nullptr) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;   // vector of 8 elements
  const bool live = i < n_vec;
  float v[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  if (live) unpack8(reinterpret_cast<const bf16x8*>(x)[i], v);
  float amax = 0.f;
#pragma unroll
  for (int j = 0; j < 8; ++j) amax = fmaxf(amax, fabsf(v[j]));
  amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
  amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
  if (!live) return;
  // row_exp: one given exponent per row (float8 row-wise scaling with power-of-two scales) instead of one per block
  const uint32_t e = row_exp != nullptr ? (uint32_t)row_exp[(i * 8) / C] : e8m0_rceil(amax);
  const float inv = e8m0_inverse(e);
  const uint32_t lo = to_e4m3x4(v[0] * inv, v[1] * inv, v[2] * inv, v[3] * inv);
  const uint32_t hi = to_e4m3x4(v[4] * inv, v[5] * inv, v[6] * inv, v[7] * inv);
  if (kFake) {
    const float s = e8m0_to_float(e);
    float r[8];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      r[j] = from_e4m3((lo >> (8 * j)) & 0xffu) * s;
      r[4 + j] = from_e4m3((hi >> (8 * j)) & 0xffu) * s;
    }
    reinterpret_cast<bf16x8*>(fake)[i] = pack8(r);
  } else {
    reinterpret_cast<uint2*>(data)[i] = make_uint2(lo, hi);
    if ((i & 3) == 0) {
      if (kTiled) {
        const int64_t el = i * 8;
        const int64_t row = el / C;
        const int blk = (int)(el % C) >> 5;
        const int r = (int)(row & 127);
        const int64_t atom = (row >> 7) * (C >> 7) + (blk >> 2);
        scales[atom * 512 + (r & 31) * 16 + (r >> 5) * 4 + (blk & 3)] = (uint8_t)e;
      } else {
        scales[i >> 2] = (uint8_t)e;   // element index 8 i -> block 8 i / 32
      }
    }
  }
}

// ---- axis 0: one thread owns a column pair over a block of 32 rows
template <bool kFake>
__global__ void mx_colwise_kernel(const __nv_bfloat16* __restrict__ x, uint8_t* __restrict__ data,
                                  uint8_t* __restrict__ scales, __nv_bfloat16* __restrict__ fake, int R, int C) {
  const int c2 = blockIdx.x * blockDim.x + threadIdx.x;   // column pair
  const int rb = blockIdx.y;                               // block of 32 rows
  if (c2 * 2 >= C) return;
  const int r0 = rb * 32;
  const int rows = min(32, R - r0);
  float2 v[32];
  float a0 = 0.f, a1 = 0.f;
#pragma unroll
  for (int r = 0; r < 32; ++r) {
    v[r] = make_float2(0.f, 0.f);
    if (r < rows) v[r] = __bfloat1622float2(reinterpret_cast<const __nv_bfloat162*>(x + (int64_t)(r0 + r) * C)[c2]);
    a0 = fmaxf(a0, fabsf(v[r].x));
    a1 = fmaxf(a1, fabsf(v[r].y));
  }
  const uint32_t e0 = e8m0_rceil(a0), e1 = e8m0_rceil(a1);
  const float i0 = e8m0_inverse(e0), i1 = e8m0_inverse(e1);
  const float s0 = e8m0_to_float(e0), s1 = e8m0_to_float(e1);
#pragma unroll
  for (int r = 0; r < 32; ++r) {
    if (r >= rows) break;
    const uint32_t q = __nv_cvt_float2_to_fp8x2(make_float2(v[r].x * i0, v[r].y * i1), __NV_SATFINITE, __NV_E4M3);
    if (kFake) {
      reinterpret_cast<__nv_bfloat162*>(fake + (int64_t)(r0 + r) * C)[c2] =
          __floats2bfloat162_rn(from_e4m3(q & 0xffu) * s0, from_e4m3((q >> 8) & 0xffu) * s1);
    } else {
      reinterpret_cast<uint16_t*>(data + (int64_t)(r0 + r) * C)[c2] = (uint16_t)q;
    }
  }
  if (!kFake) {
    scales[(int64_t)rb * C + 2 * c2] = (uint8_t)e0;
    scales[(int64_t)rb * C + 2 * c2 + 1] = (uint8_t)e1;
  }
}

// ---- transposing quantiser: x [R, C] -> data [C, R] e4m3, scaled along R (blocks of 32 rows of x
// become blocks of 32 contiguous bytes of an output row), scales in the GEMM's tiled layout over
// (rows = C, contraction = R).  One CTA moves a tile of 128 rows x 64 columns through shared
// memory (16-byte chunks, XOR-swizzled by the row block so that the column reads below do not
// collide); thread (c, b) then owns column c over row block b and writes 32 contiguous bytes, the
// four threads of a column one 128-byte line.
// kBoth: the same tile also yields the row-wise form (data_row [R, C] scaled along C, tiled scales over rows = R,
// contraction = C), so an operand that two GEMMs contract over different dimensions is read from memory once:
// thread (r, h) owns the 32 columns of half h of tile row r.
constexpr int kTqRows = 128, kTqCols = 64;
template <bool kBoth>
__global__ void __launch_bounds__(256)
mx_transpose_tiled_kernel(const __nv_bfloat16* __restrict__ x, uint8_t* __restrict__ data, uint8_t* __restrict__ scales,
                          uint8_t* __restrict__ data_row, uint8_t* __restrict__ scales_row, int R, int C,
                          const uint8_t* __restrict__ col_exp = nullptr) {
  __shared__ __align__(16) uint8_t tile[kTqRows * kTqCols * 2];
  const int r0 = blockIdx.y * kTqRows, c0 = blockIdx.x * kTqCols;
  // load: 1024 chunks of 8 elements, 4 per thread (row = chunk / 8)
#pragma unroll
  for (int u = 0; u < 4; ++u) {
    const int ch = threadIdx.x + u * 256;
    const int r = ch >> 3, cc = ch & 7;
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (c0 + cc * 8 < C) v = *reinterpret_cast<const uint4*>(x + (int64_t)(r0 + r) * C + c0 + cc * 8);
    *reinterpret_cast<uint4*>(tile + r * 128 + ((cc ^ ((r >> 5) * 2)) << 4)) = v;
  }
  __syncthreads();
  if (kBoth) {
    const int r = threadIdx.x >> 1, h = threadIdx.x & 1;
    if (c0 + h * 32 < C) {
      float v[32];
      float amax = 0.f;
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const int cc = h * 4 + q;
        const uint4 raw = *reinterpret_cast<const uint4*>(tile + r * 128 + ((cc ^ ((r >> 5) * 2)) << 4));
        unpack8(*reinterpret_cast<const bf16x8*>(&raw), *reinterpret_cast<float(*)[8]>(v + q * 8));
      }
#pragma unroll
      for (int i = 0; i < 32; ++i) amax = fmaxf(amax, fabsf(v[i]));
      const uint32_t e = e8m0_rceil(amax);
      const float inv = e8m0_inverse(e);
      uint32_t w[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) w[i] = to_e4m3x4(v[4 * i] * inv, v[4 * i + 1] * inv, v[4 * i + 2] * inv, v[4 * i + 3] * inv);
      uint4* dst = reinterpret_cast<uint4*>(data_row + (int64_t)(r0 + r) * C + c0 + h * 32);
      dst[0] = make_uint4(w[0], w[1], w[2], w[3]);
      dst[1] = make_uint4(w[4], w[5], w[6], w[7]);
      const int row = r0 + r;
      const int blk = (c0 >> 5) + h;
      const int64_t atom = (int64_t)(row >> 7) * (C >> 7) + (blk >> 2);
      scales_row[atom * 512 + (row & 31) * 16 + ((row & 127) >> 5) * 4 + (blk & 3)] = (uint8_t)e;
    }
  }
  const int b = threadIdx.x & 3, c = threadIdx.x >> 2;
  if (c0 + c >= C) return;
  const int cc = (c >> 3) ^ (b * 2);
  const uint8_t* src = tile + (b * 32) * 128 + (cc << 4) + (c & 7) * 2;
  float v[32];
  float amax = 0.f;
#pragma unroll
  for (int i = 0; i < 32; ++i) {
    v[i] = __bfloat162float(*reinterpret_cast<const __nv_bfloat16*>(src + i * 128));
    amax = fmaxf(amax, fabsf(v[i]));
  }
  // col_exp: one given exponent per column of x, i.e. per output row (float8 row-wise scaling, power-of-two scales)
  const uint32_t e = col_exp != nullptr ? (uint32_t)col_exp[c0 + c] : e8m0_rceil(amax);
  const float inv = e8m0_inverse(e);
  uint32_t w[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) w[i] = to_e4m3x4(v[4 * i] * inv, v[4 * i + 1] * inv, v[4 * i + 2] * inv, v[4 * i + 3] * inv);
  uint4* dst = reinterpret_cast<uint4*>(data + (int64_t)(c0 + c) * R + r0 + b * 32);
  dst[0] = make_uint4(w[0], w[1], w[2], w[3]);
  dst[1] = make_uint4(w[4], w[5], w[6], w[7]);
  const int row = c0 + c;
  const int64_t atom = (int64_t)(row >> 7) * (R >> 7) + blockIdx.y;
  scales[atom * 512 + (row & 31) * 16 + ((row & 127) >> 5) * 4 + b] = (uint8_t)e;
}

__global__ void mx_dequant_kernel(const uint8_t* __restrict__ data, const uint8_t* __restrict__ scales,
                                  __nv_bfloat16* __restrict__ out, int64_t n_vec, int C, int axis) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;   // 8 elements
  if (i >= n_vec) return;
  const uint2 q = reinterpret_cast<const uint2*>(data)[i];
  const int64_t el = i * 8;
  const int64_t row = el / C;
  const int col = (int)(el % C);
  float r[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const uint32_t byte = ((j < 4 ? q.x : q.y) >> (8 * (j & 3))) & 0xffu;
    const uint32_t e = axis == 1 ? scales[el >> 5] : scales[(row >> 5) * C + col + j];
    r[j] = from_e4m3(byte) * e8m0_to_float(e);
  }
  reinterpret_cast<bf16x8*>(out)[i] = pack8(r);
}

// ---- float8 row-wise: one warp per row, scale = amax / 448 (fp32)
template <bool kFake>
__global__ void f8_rowwise_kernel(const __nv_bfloat16* __restrict__ x, uint8_t* __restrict__ data,
                                  float* __restrict__ scales, __nv_bfloat16* __restrict__ fake, int64_t R, int C) {
  const int64_t row = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (row >= R) return;
  const bf16x8* src = reinterpret_cast<const bf16x8*>(x + row * C);
  float amax = 0.f;
  for (int i = lane; i < C / 8; i += 32) {
    float v[8];
    unpack8(src[i], v);
#pragma unroll
    for (int j = 0; j < 8; ++j) amax = fmaxf(amax, fabsf(v[j]));
  }
  amax = warp_max(amax);
  const float scale = __fdiv_rn(fmaxf(amax, 1e-12f), kE4M3Max);
  for (int i = lane; i < C / 8; i += 32) {
    float v[8];
    unpack8(src[i], v);
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] = __fdiv_rn(v[j], scale);   // the exact quotient, as the PyTorch restatement computes it
    const uint32_t lo = to_e4m3x4(v[0], v[1], v[2], v[3]);
    const uint32_t hi = to_e4m3x4(v[4], v[5], v[6], v[7]);
    if (kFake) {
      float r[8];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        r[j] = from_e4m3((lo >> (8 * j)) & 0xffu) * scale;
        r[4 + j] = from_e4m3((hi >> (8 * j)) & 0xffu) * scale;
      }
      reinterpret_cast<bf16x8*>(fake + row * C)[i] = pack8(r);
    } else {
      reinterpret_cast<uint2*>(data + row * C)[i] = make_uint2(lo, hi);
    }
  }
  if (!kFake && lane == 0) scales[row] = scale;
}

static void check_q_input(const at::Tensor& x, int64_t axis) {
  TORCH_CHECK(x.is_cuda() && x.scalar_type() == at::kBFloat16 && x.dim() == 2 && x.is_contiguous(),
              "quantize: a contiguous bf16 [R, C] CUDA tensor is expected");
  TORCH_CHECK(axis == 0 || axis == 1, "quantize: axis must be 0 or 1");
  if (axis == 1) {
    TORCH_CHECK(x.size(1) % 32 == 0, "mxfp8 along the last dimension needs C % 32 == 0");
  } else {
    TORCH_CHECK(x.size(1) % 8 == 0, "mxfp8 along the first dimension needs C % 8 == 0");
  }
}

template <bool kFake>
static void launch_mx(const at::Tensor& x, int64_t axis, uint8_t* data, uint8_t* scales, __nv_bfloat16* fake) {
  const int64_t R = x.size(0);
  const int C = (int)x.size(1);
  auto stream = at::cuda::getCurrentCUDAStream();
  auto xp = reinterpret_cast<const __nv_bfloat16*>(x.data_ptr());
  if (R == 0 || C == 0) return;
  if (axis == 1) {
    const int64_t n_vec = R * C / 8;
    mx_rowwise_kernel<kFake><<<(unsigned)((n_vec + 255) / 256), 256, 0, stream>>>(xp, data, scales, fake, n_vec, C);
  } else {
    dim3 grid((unsigned)((C / 2 + 127) / 128), (unsigned)((R + 31) / 32));
    mx_colwise_kernel<kFake><<<grid, 128, 0, stream>>>(xp, data, scales, fake, (int)R, C);
  }
  C10_CUDA_KERNEL_LAUNCH_CHECK();
}

std::tuple<at::Tensor, at::Tensor> mxfp8_quantize(const at::Tensor& x, int64_t axis) {
  check_q_input(x, axis);
  c10::cuda::CUDAGuard guard(x.device());
  const int64_t R = x.size(0), C = x.size(1);
  auto data = at::empty({R, C}, x.options().dtype(at::kByte));
  auto scales = axis == 1 ? at::empty({R, C / 32}, x.options().dtype(at::kByte))
                          : at::empty({(R + 31) / 32, C}, x.options().dtype(at::kByte));
  launch_mx<false>(x, axis, data.data_ptr<uint8_t>(), scales.data_ptr<uint8_t>(), nullptr);
  return {data, scales};
}

// Row-wise MXFP8 with the scale layout of the block-scaled GEMM (`gemm_mxfp8`); C % 128 == 0.
std::tuple<at::Tensor, at::Tensor> mxfp8_quantize_tiled(const at::Tensor& x) {
  check_q_input(x, 1);
  TORCH_CHECK(x.size(1) % 128 == 0, "mxfp8_quantize_tiled: the contraction dimension must be a multiple of 128");
  c10::cuda::CUDAGuard guard(x.device());
  const int64_t R = x.size(0), C = x.size(1);
  auto data = at::empty({R, C}, x.options().dtype(at::kByte));
  const int64_t n_sf = (R + 127) / 128 * (C / 128) * 512;   // rows past R keep scale byte 0 (2^-127), never NaN
  auto scales = R % 128 == 0 ? at::empty({n_sf}, x.options().dtype(at::kByte)) : at::zeros({n_sf}, x.options().dtype(at::kByte));
  const int64_t n_vec = R * C / 8;
  if (n_vec > 0)
    mx_rowwise_kernel<false, true><<<(unsigned)((n_vec + 255) / 256), 256, 0, at::cuda::getCurrentCUDAStream()>>>(
        reinterpret_cast<const __nv_bfloat16*>(x.data_ptr()), data.data_ptr<uint8_t>(), scales.data_ptr<uint8_t>(), nullptr,
        n_vec, (int)C);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  return {data, scales};
}

// Column-wise MXFP8 of x [R, C] written transposed, as a K-major GEMM operand: data [C, R] scaled
// along R, with the tiled scale layout over (rows = C, contraction = R); R % 128 == 0, C % 8 == 0.
std::tuple<at::Tensor, at::Tensor> mxfp8_quantize_tiled_t(const at::Tensor& x) {
  check_q_input(x, 0);
  TORCH_CHECK(x.size(0) % 128 == 0, "mxfp8_quantize_tiled_t: the contraction dimension (rows) must be a multiple of 128");
  c10::cuda::CUDAGuard guard(x.device());
  const int64_t R = x.size(0), C = x.size(1);
  auto data = at::empty({C, R}, x.options().dtype(at::kByte));
  const int64_t n_sf = (C + 127) / 128 * (R / 128) * 512;
  auto scales = C % 128 == 0 ? at::empty({n_sf}, x.options().dtype(at::kByte)) : at::zeros({n_sf}, x.options().dtype(at::kByte));
  if (R > 0 && C > 0) {
    dim3 grid((unsigned)((C + kTqCols - 1) / kTqCols), (unsigned)(R / kTqRows));
    mx_transpose_tiled_kernel<false><<<grid, 256, 0, at::cuda::getCurrentCUDAStream()>>>(
        reinterpret_cast<const __nv_bfloat16*>(x.data_ptr()), data.data_ptr<uint8_t>(), scales.data_ptr<uint8_t>(), nullptr,
        nullptr, (int)R, (int)C);
    C10_CUDA_KERNEL_LAUNCH_CHECK();
  }
  return {data, scales};
}

// Both MXFP8 forms of x [R, C] from one read: (row-wise data [R, C], its tiled scales, transposed data [C, R] scaled
// along R, its tiled scales), i.e. mxfp8_quantize_tiled(x) and mxfp8_quantize_tiled_t(x).  R % 128 == 0, C % 128 == 0.
std::tuple<at::Tensor, at::Tensor, at::Tensor, at::Tensor> mxfp8_quantize_tiled_both(const at::Tensor& x) {
  check_q_input(x, 0);
  TORCH_CHECK(x.size(0) % 128 == 0 && x.size(1) % 128 == 0, "mxfp8_quantize_tiled_both: both dimensions must be multiples of 128");
  c10::cuda::CUDAGuard guard(x.device());
  const int64_t R = x.size(0), C = x.size(1);
  auto bopt = x.options().dtype(at::kByte);
  auto data_row = at::empty({R, C}, bopt);
  auto scales_row = at::empty({R / 128 * (C / 128) * 512}, bopt);
  auto data_t = at::empty({C, R}, bopt);
  auto scales_t = at::empty({C / 128 * (R / 128) * 512}, bopt);
  if (R > 0 && C > 0) {
    dim3 grid((unsigned)(C / kTqCols), (unsigned)(R / kTqRows));
    mx_transpose_tiled_kernel<true><<<grid, 256, 0, at::cuda::getCurrentCUDAStream()>>>(
        reinterpret_cast<const __nv_bfloat16*>(x.data_ptr()), data_t.data_ptr<uint8_t>(), scales_t.data_ptr<uint8_t>(),
        data_row.data_ptr<uint8_t>(), scales_row.data_ptr<uint8_t>(), (int)R, (int)C);
    C10_CUDA_KERNEL_LAUNCH_CHECK();
  }
  return {data_row, scales_row, data_t, scales_t};
}

// Float8 row-wise scaling with power-of-two scales, in the operand format of the block-scaled GEMM: every 32-element
// block of a row carries the row's exponent `exps[row]` (e8m0).  x [R, C], C % 128 == 0.
std::tuple<at::Tensor, at::Tensor> float8_pow2_quantize_tiled(const at::Tensor& x, const at::Tensor& exps) {
  check_q_input(x, 1);
  const int64_t R = x.size(0), C = x.size(1);
  TORCH_CHECK(C % 128 == 0, "float8_pow2_quantize_tiled: the contraction dimension must be a multiple of 128");
  TORCH_CHECK(exps.is_cuda() && exps.scalar_type() == at::kByte && exps.is_contiguous() && exps.numel() == R);
  c10::cuda::CUDAGuard guard(x.device());
  auto data = at::empty({R, C}, x.options().dtype(at::kByte));
  const int64_t n_sf = (R + 127) / 128 * (C / 128) * 512;
  auto scales = R % 128 == 0 ? at::empty({n_sf}, x.options().dtype(at::kByte)) : at::zeros({n_sf}, x.options().dtype(at::kByte));
  const int64_t n_vec = R * C / 8;
  if (n_vec > 0)
    mx_rowwise_kernel<false, true><<<(unsigned)((n_vec + 255) / 256), 256, 0, at::cuda::getCurrentCUDAStream()>>>(
        reinterpret_cast<const __nv_bfloat16*>(x.data_ptr()), data.data_ptr<uint8_t>(), scales.data_ptr<uint8_t>(), nullptr,
        n_vec, (int)C, exps.data_ptr<uint8_t>());
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  return {data, scales};
}

// The same for an operand contracted over its rows: x [R, C] -> data [C, R], output row c scaled by exps[c]; R % 128 == 0.
std::tuple<at::Tensor, at::Tensor> float8_pow2_quantize_tiled_t(const at::Tensor& x, const at::Tensor& exps) {
  check_q_input(x, 0);
  const int64_t R = x.size(0), C = x.size(1);
  TORCH_CHECK(R % 128 == 0, "float8_pow2_quantize_tiled_t: the contraction dimension (rows) must be a multiple of 128");
  TORCH_CHECK(exps.is_cuda() && exps.scalar_type() == at::kByte && exps.is_contiguous() && exps.numel() == C);
  c10::cuda::CUDAGuard guard(x.device());
  auto data = at::empty({C, R}, x.options().dtype(at::kByte));
  const int64_t n_sf = (C + 127) / 128 * (R / 128) * 512;
  auto scales = C % 128 == 0 ? at::empty({n_sf}, x.options().dtype(at::kByte)) : at::zeros({n_sf}, x.options().dtype(at::kByte));
  if (R > 0 && C > 0) {
    dim3 grid((unsigned)((C + kTqCols - 1) / kTqCols), (unsigned)(R / kTqRows));
    mx_transpose_tiled_kernel<false><<<grid, 256, 0, at::cuda::getCurrentCUDAStream()>>>(
        reinterpret_cast<const __nv_bfloat16*>(x.data_ptr()), data.data_ptr<uint8_t>(), scales.data_ptr<uint8_t>(), nullptr,
        nullptr, (int)R, (int)C, exps.data_ptr<uint8_t>());
    C10_CUDA_KERNEL_LAUNCH_CHECK();
  }
  return {data, scales};
}

at::Tensor mxfp8_fake_quant(const at::Tensor& x, int64_t axis) {
  check_q_input(x, axis);
  c10::cuda::CUDAGuard guard(x.device());
  auto out = at::empty_like(x);
  launch_mx<true>(x, axis, nullptr, nullptr, reinterpret_cast<__nv_bfloat16*>(out.data_ptr()));
  return out;
}

at::Tensor mxfp8_dequantize(const at::Tensor& data, const at::Tensor& scales, int64_t axis) {
  TORCH_CHECK(data.is_cuda() && data.scalar_type() == at::kByte && data.dim() == 2 && data.is_contiguous());
  TORCH_CHECK(scales.is_cuda() && scales.scalar_type() == at::kByte && scales.is_contiguous());
  TORCH_CHECK(data.size(1) % 8 == 0 && (axis == 0 || data.size(1) % 32 == 0));
  c10::cuda::CUDAGuard guard(data.device());
  auto out = at::empty({data.size(0), data.size(1)}, data.options().dtype(at::kBFloat16));
  const int64_t n_vec = data.numel() / 8;
  if (n_vec == 0) return out;
  mx_dequant_kernel<<<(unsigned)((n_vec + 255) / 256), 256, 0, at::cuda::getCurrentCUDAStream()>>>(
      data.data_ptr<uint8_t>(), scales.data_ptr<uint8_t>(), reinterpret_cast<__nv_bfloat16*>(out.data_ptr()), n_vec,
      (int)data.size(1), (int)axis);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  return out;
}

std::tuple<at::Tensor, at::Tensor> float8_rowwise_quantize(const at::Tensor& x) {
  check_q_input(x, 0);
  c10::cuda::CUDAGuard guard(x.device());
  const int64_t R = x.size(0);
  auto data = at::empty({R, x.size(1)}, x.options().dtype(at::kByte));
  auto scales = at::empty({R}, x.options().dtype(at::kFloat));
  if (R > 0)
    f8_rowwise_kernel<false><<<(unsigned)((R * 32 + 255) / 256), 256, 0, at::cuda::getCurrentCUDAStream()>>>(
        reinterpret_cast<const __nv_bfloat16*>(x.data_ptr()), data.data_ptr<uint8_t>(), scales.data_ptr<float>(), nullptr, R,
        (int)x.size(1));
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  return {data, scales};
}

at::Tensor float8_rowwise_fake_quant(const at::Tensor& x) {
  check_q_input(x, 0);
  c10::cuda::CUDAGuard guard(x.device());
  auto out = at::empty_like(x);
  const int64_t R = x.size(0);
  if (R > 0)
    f8_rowwise_kernel<true><<<(unsigned)((R * 32 + 255) / 256), 256, 0, at::cuda::getCurrentCUDAStream()>>>(
        reinterpret_cast<const __nv_bfloat16*>(x.data_ptr()), nullptr, nullptr,
        reinterpret_cast<__nv_bfloat16*>(out.data_ptr()), R, (int)x.size(1));
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  return out;
}

}  // namespace tb200
