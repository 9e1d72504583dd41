// Multi-head latent attention: rotary embedding of the decoupled q / k parts and assembly of the attention operands
// in one pass (forward) and its transpose (backward).
//
//   q  [T, H, dn + dr]   output of the query up-projection        -> qf [T, H, dn + dr] = [q_nope | rope(q_pe)]
//   kv [T, H, dn + dv]   output of the key / value up-projection   -> kf [T, H, dn + dr] = [k_nope | rope(k_pe)]
//   k_pe [T, dr]         rotary key shared by all heads (a column     v  [T, H, dv]      (contiguous)
//                        slice of the compressed projection)
//
// Replaces two rotary launches, two concatenations and the broadcast of k_pe over the heads.  The rotation pairs
// adjacent elements (2i, 2i + 1); `table[P, dr]` holds cos | sin in fp32.  bf16, 16-byte vectors: dn, dr and dv
// must be multiples of 8.  A position outside the table is clamped and reported in the status word.
#include <ATen/ATen.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/library.h>

#include "common.cuh"

namespace tb200 {
int* status_word_ptr();   // elementwise.cu: the status word that `status()` reports

namespace {

using bf16 = __nv_bfloat16;

__device__ __forceinline__ void rotate8(float (&f)[8], const float* __restrict__ cs, int half, int pair0, float sign) {
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float c = cs[pair0 + j], s = sign * cs[half + pair0 + j];
    const float a = f[2 * j], b = f[2 * j + 1];
    f[2 * j] = a * c - b * s;
    f[2 * j + 1] = a * s + b * c;
  }
}

__device__ __forceinline__ int64_t checked_pos(const int64_t* positions, int64_t row, int P, int* status) {
  int64_t pos = positions[row];
  if (pos < 0 || pos >= P) {
    atomicOr(status, kStatusRopePositionOutOfRange);
    pos = pos < 0 ? 0 : P - 1;
  }
  return pos;
}

__global__ void __launch_bounds__(256)
mla_assemble_fwd_kernel(const bf16* __restrict__ q, const bf16* __restrict__ kv, const bf16* __restrict__ k_pe,
                        int64_t k_pe_stride, const float* __restrict__ table, const int64_t* __restrict__ positions,
                        bf16* __restrict__ qf, bf16* __restrict__ kf, bf16* __restrict__ v, int64_t T_, int H, int dn,
                        int dr, int dv, int P, int* __restrict__ status) {
  const int nqk = (dn + dr) / 8, nv = dv / 8, per_head = 2 * nqk + nv, half = dr / 2;
  const int64_t total = T_ * H * per_head;
  for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (int64_t)gridDim.x * blockDim.x) {
    const int it = (int)(idx % per_head);
    const int64_t rh = idx / per_head;
    const int h = (int)(rh % H);
    const int64_t row = rh / H;
    const int64_t qk_off = (row * H + h) * (int64_t)(dn + dr);
    float f[8];
    if (it < nqk) {                                   // query vector
      const int e = it * 8;
      unpack8(*reinterpret_cast<const bf16x8*>(q + qk_off + e), f);
      if (e >= dn) rotate8(f, table + checked_pos(positions, row, P, status) * dr, half, (e - dn) / 2, 1.f);
      *reinterpret_cast<bf16x8*>(qf + qk_off + e) = pack8(f);
    } else if (it < 2 * nqk) {                        // key vector: nope part of this head, or the shared rotary part
      const int e = (it - nqk) * 8;
      if (e < dn) {
        *reinterpret_cast<bf16x8*>(kf + qk_off + e) =
            *reinterpret_cast<const bf16x8*>(kv + (row * H + h) * (int64_t)(dn + dv) + e);
      } else {
        unpack8(*reinterpret_cast<const bf16x8*>(k_pe + row * k_pe_stride + (e - dn)), f);
        rotate8(f, table + checked_pos(positions, row, P, status) * dr, half, (e - dn) / 2, 1.f);
        *reinterpret_cast<bf16x8*>(kf + qk_off + e) = pack8(f);
      }
    } else {                                          // value vector
      const int e = (it - 2 * nqk) * 8;
      *reinterpret_cast<bf16x8*>(v + (row * H + h) * (int64_t)dv + e) =
          *reinterpret_cast<const bf16x8*>(kv + (row * H + h) * (int64_t)(dn + dv) + dn + e);
    }
  }
}

__global__ void __launch_bounds__(256)
mla_assemble_bwd_kernel(const bf16* __restrict__ dqf, const bf16* __restrict__ dkf, const bf16* __restrict__ dvv,
                        const float* __restrict__ table, const int64_t* __restrict__ positions, bf16* __restrict__ dq,
                        bf16* __restrict__ dkv, bf16* __restrict__ dk_pe, int64_t T_, int H, int dn, int dr, int dv,
                        int P, int* __restrict__ status) {
  const int nqk = (dn + dr) / 8, nkn = dn / 8, nv = dv / 8, per_head = nqk + nkn + nv, half = dr / 2, npe = dr / 8;
  const int64_t head_items = T_ * H * per_head;
  const int64_t total = head_items + T_ * npe;
  for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (int64_t)gridDim.x * blockDim.x) {
    float f[8];
    if (idx >= head_items) {                          // gradient of the shared rotary key: sum over the heads
      const int64_t r = idx - head_items;
      const int it = (int)(r % npe);
      const int64_t row = r / npe;
      float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
      for (int h = 0; h < H; ++h) {
        unpack8(*reinterpret_cast<const bf16x8*>(dkf + (row * H + h) * (int64_t)(dn + dr) + dn + it * 8), f);
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] += f[j];
      }
      rotate8(acc, table + checked_pos(positions, row, P, status) * dr, half, it * 4, -1.f);
      *reinterpret_cast<bf16x8*>(dk_pe + row * (int64_t)dr + it * 8) = pack8(acc);
      continue;
    }
    const int it = (int)(idx % per_head);
    const int64_t rh = idx / per_head;
    const int h = (int)(rh % H);
    const int64_t row = rh / H;
    const int64_t qk_off = (row * H + h) * (int64_t)(dn + dr), kv_off = (row * H + h) * (int64_t)(dn + dv);
    if (it < nqk) {
      const int e = it * 8;
      unpack8(*reinterpret_cast<const bf16x8*>(dqf + qk_off + e), f);
      if (e >= dn) rotate8(f, table + checked_pos(positions, row, P, status) * dr, half, (e - dn) / 2, -1.f);
      *reinterpret_cast<bf16x8*>(dq + qk_off + e) = pack8(f);
    } else if (it < nqk + nkn) {
      const int e = (it - nqk) * 8;
      *reinterpret_cast<bf16x8*>(dkv + kv_off + e) = *reinterpret_cast<const bf16x8*>(dkf + qk_off + e);
    } else {
      const int e = (it - nqk - nkn) * 8;
      *reinterpret_cast<bf16x8*>(dkv + kv_off + dn + e) =
          *reinterpret_cast<const bf16x8*>(dvv + (row * H + h) * (int64_t)dv + e);
    }
  }
}

void check3(const at::Tensor& t, const char* name) {
  TORCH_CHECK(t.is_cuda() && t.scalar_type() == at::kBFloat16 && t.dim() == 3 && t.is_contiguous(), "mla_assemble: ", name,
              " must be a contiguous [T, H, D] bf16 CUDA tensor");
}

int launch_grid(int64_t total) {
  return (int)std::max<int64_t>(1, std::min<int64_t>((total + 255) / 256, (int64_t)num_sms() * 16));
}

}  // namespace

// Returns (qf, kf, v).  `k_pe` is [T, dr] with unit column stride (its rows may be strided).
std::tuple<at::Tensor, at::Tensor, at::Tensor> mla_assemble_fwd(const at::Tensor& q, const at::Tensor& kv,
                                                                const at::Tensor& k_pe, const at::Tensor& table,
                                                                const at::Tensor& positions, int64_t dn, int64_t dr,
                                                                int64_t dv) {
  check3(q, "q"); check3(kv, "kv");
  const int64_t T_ = q.size(0);
  const int H = (int)q.size(1);
  TORCH_CHECK(q.size(2) == dn + dr && kv.size(0) == T_ && kv.size(1) == H && kv.size(2) == dn + dv);
  TORCH_CHECK(dn % 8 == 0 && dr % 8 == 0 && dv % 8 == 0, "mla_assemble: head dimensions must be multiples of 8");
  TORCH_CHECK(k_pe.is_cuda() && k_pe.scalar_type() == at::kBFloat16 && k_pe.dim() == 2 && k_pe.size(0) == T_ &&
                  k_pe.size(1) == dr && k_pe.stride(1) == 1 && (k_pe.stride(0) * 2) % 16 == 0 &&
                  (reinterpret_cast<uintptr_t>(k_pe.data_ptr()) & 15) == 0,
              "mla_assemble: k_pe must be [T, dr] bf16 with 16-byte aligned rows");
  TORCH_CHECK(table.is_cuda() && table.scalar_type() == at::kFloat && table.is_contiguous() && table.size(1) == dr);
  TORCH_CHECK(positions.is_cuda() && positions.scalar_type() == at::kLong && positions.is_contiguous() &&
              positions.numel() == T_);
  c10::cuda::CUDAGuard guard(q.device());
  auto qf = at::empty_like(q);
  auto kf = at::empty_like(q);
  auto v = at::empty({T_, H, dv}, q.options());
  if (T_ == 0) return {qf, kf, v};
  const int64_t total = T_ * H * (2 * (dn + dr) / 8 + dv / 8);
  mla_assemble_fwd_kernel<<<launch_grid(total), 256, 0, at::cuda::getCurrentCUDAStream()>>>(
      reinterpret_cast<const bf16*>(q.data_ptr()), reinterpret_cast<const bf16*>(kv.data_ptr()),
      reinterpret_cast<const bf16*>(k_pe.data_ptr()), k_pe.stride(0), table.data_ptr<float>(),
      positions.data_ptr<int64_t>(), reinterpret_cast<bf16*>(qf.data_ptr()), reinterpret_cast<bf16*>(kf.data_ptr()),
      reinterpret_cast<bf16*>(v.data_ptr()), T_, H, (int)dn, (int)dr, (int)dv, (int)table.size(0), status_word_ptr());
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  return {qf, kf, v};
}

// Returns (dq [T, H, dn + dr], dkv [T, H, dn + dv], dk_pe [T, dr]).
std::tuple<at::Tensor, at::Tensor, at::Tensor> mla_assemble_bwd(const at::Tensor& dqf, const at::Tensor& dkf,
                                                                const at::Tensor& dv_, const at::Tensor& table,
                                                                const at::Tensor& positions, int64_t dn, int64_t dr,
                                                                int64_t dv) {
  check3(dqf, "dqf"); check3(dkf, "dkf"); check3(dv_, "dv");
  const int64_t T_ = dqf.size(0);
  const int H = (int)dqf.size(1);
  TORCH_CHECK(dqf.size(2) == dn + dr && dkf.sizes() == dqf.sizes() && dv_.size(0) == T_ && dv_.size(1) == H && dv_.size(2) == dv);
  TORCH_CHECK(dn % 8 == 0 && dr % 8 == 0 && dv % 8 == 0);
  TORCH_CHECK(table.is_cuda() && table.scalar_type() == at::kFloat && table.is_contiguous() && table.size(1) == dr);
  TORCH_CHECK(positions.is_cuda() && positions.scalar_type() == at::kLong && positions.is_contiguous() &&
              positions.numel() == T_);
  c10::cuda::CUDAGuard guard(dqf.device());
  auto dq = at::empty_like(dqf);
  auto dkv = at::empty({T_, H, dn + dv}, dqf.options());
  auto dk_pe = at::empty({T_, dr}, dqf.options());
  if (T_ == 0) return {dq, dkv, dk_pe};
  const int64_t total = T_ * H * ((dn + dr) / 8 + dn / 8 + dv / 8) + T_ * (dr / 8);
  mla_assemble_bwd_kernel<<<launch_grid(total), 256, 0, at::cuda::getCurrentCUDAStream()>>>(
      reinterpret_cast<const bf16*>(dqf.data_ptr()), reinterpret_cast<const bf16*>(dkf.data_ptr()),
      reinterpret_cast<const bf16*>(dv_.data_ptr()), table.data_ptr<float>(), positions.data_ptr<int64_t>(),
      reinterpret_cast<bf16*>(dq.data_ptr()), reinterpret_cast<bf16*>(dkv.data_ptr()),
      reinterpret_cast<bf16*>(dk_pe.data_ptr()), T_, H, (int)dn, (int)dr, (int)dv, (int)table.size(0),
      status_word_ptr());
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  return {dq, dkv, dk_pe};
}

}  // namespace tb200
