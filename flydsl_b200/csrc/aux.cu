// Bandwidth-bound helpers around the GEMM stages: row gather into sorted order,
// top-k reduce, 1x128 activation quantiser, weight (un)shuffle.
#include <algorithm>

#include "common.cuh"

namespace flymoe {

// ---------------------------------------------------------------------------- gather
// One warp per sorted row, 16 bytes per lane per step.
__global__ void __launch_bounds__(256)
gather_rows_kernel(const uint4* __restrict__ src, uint4* __restrict__ dst,
                   const int* __restrict__ sorted_ids, const int* __restrict__ num_valid_ids,
                   int num_tokens, int topk, int row_vec, int src_layout, int max_rows) {
  const int lane = threadIdx.x & 31;
  const int warps_per_block = blockDim.x >> 5;
  const int valid = min(__ldg(num_valid_ids), max_rows);
  for (int r = blockIdx.x * warps_per_block + (threadIdx.x >> 5); r < valid;
       r += gridDim.x * warps_per_block) {
    const int id = __ldg(sorted_ids + r);
    const int t = id_token(id), s = id_slot(id);
    uint4* d = dst + size_t(r) * row_vec;
    if (t < num_tokens && s < topk) {
      const size_t srow = src_layout == FLYMOE_ROWS_BY_TOKEN ? size_t(t)
                        : src_layout == FLYMOE_ROWS_BY_SLOT ? size_t(s) * num_tokens + t : size_t(t) * topk + s;
      const uint4* p = src + srow * row_vec;
      for (int i = lane; i < row_vec; i += 32) d[i] = __ldg(p + i);
    } else {
      for (int i = lane; i < row_vec; i += 32) d[i] = make_uint4(0, 0, 0, 0);
    }
  }
}

// ---------------------------------------------------------------------------- dispatch
// One warp per (token, slot) row in this rank's expert-sorted order.  The row's e4m3 bytes and its
// fp32 scales are stored where the per-expert tables say -- normally into the operand
// buffers of the rank that owns the expert, at the row's final position in that rank's block-padded
// layout, so the receiver neither sorts nor gathers.  dst_*[e] is the address row 0 of THIS rank's
// order would have; row r lands r * stride bytes further.
__global__ void __launch_bounds__(256)
dispatch_rows_kernel(const uint4* __restrict__ x, const float* __restrict__ x_scale,
                     const int* __restrict__ sorted_ids, const int* __restrict__ sorted_expert_ids,
                     const int* __restrict__ num_valid_ids, const long long* __restrict__ dst_x,
                     const long long* __restrict__ dst_scale, const long long* __restrict__ pos_base,
                     long long pos_limit, int* __restrict__ status, int num_tokens, int topk, int row_vec,
                     int kblocks, int experts, int max_rows) {
  const int lane = threadIdx.x & 31;
  const int warps_per_block = blockDim.x >> 5;
  const int valid = min(__ldg(num_valid_ids), max_rows);
  // Every warp takes one contiguous piece of the sorted list (the grid is sized to be resident at once), so
  // at any moment the warps of a GPU store to all destination ranks alike.  With a grid-stride walk all GPUs
  // would work through the ranks in the same order and pile onto one receiver's links at a time.
  const int total_warps = gridDim.x * warps_per_block;
  const int piece = (valid + total_warps - 1) / total_warps;
  const int first = (blockIdx.x * warps_per_block + (threadIdx.x >> 5)) * piece;
  const int last = min(valid, first + piece);
  for (int r = first; r < last; ++r) {
    const int id = __ldg(sorted_ids + r);
    const int e = __ldg(sorted_expert_ids + r);
    const int t = id_token(id), s = id_slot(id);
    if (t >= num_tokens || s >= topk || e < 0 || e >= experts) continue;
    if (pos_base != nullptr && __ldg(pos_base + e) + r >= pos_limit) {   // would fall outside the receiver's buffer
      if (lane == 0) atomicCAS(status, 0, FLYMOE_STATUS_DISPATCH_OVERFLOW);
      continue;
    }
    const long long dst_base = __ldg(dst_x + e);
    if ((dst_base & 15) != 0) {                // the 16-byte stores below would fault: drop the row and report
      if (lane == 0) atomicCAS(status, 0, FLYMOE_STATUS_ROW_DST_MISALIGNED);
      continue;
    }
    uint4* dx = reinterpret_cast<uint4*>(dst_base + (long long)r * row_vec * 16);
    const uint4* p = x + size_t(t) * row_vec;
    // eight 16-byte loads in flight per lane before the first store: the stores cross NVLink and a loop of
    // dependent load/store pairs would leave it mostly idle
    for (int i0 = lane; i0 < row_vec; i0 += 32 * 8) {
      uint4 v[8];
#pragma unroll
      for (int j = 0; j < 8; ++j)
        if (i0 + 32 * j < row_vec) v[j] = __ldg(p + i0 + 32 * j);
#pragma unroll
      for (int j = 0; j < 8; ++j)
        if (i0 + 32 * j < row_vec) dx[i0 + 32 * j] = v[j];
    }
    float* ds = reinterpret_cast<float*>(__ldg(dst_scale + e) + (long long)r * kblocks * 4);
    const float* ps = x_scale + size_t(t) * kblocks;
    for (int i = lane; i < kblocks; i += 32) ds[i] = __ldg(ps + i);
  }
}

// ---------------------------------------------------------------------------- reduce
template <typename T> struct Vec8;
template <> struct Vec8<__half> {
  static __device__ __forceinline__ void load(const __half* p, float* f) {
    uint4 v = __ldg(reinterpret_cast<const uint4*>(p));
    const __half2* h = reinterpret_cast<const __half2*>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) { float2 x = __half22float2(h[i]); f[2 * i] = x.x; f[2 * i + 1] = x.y; }
  }
  static __device__ __forceinline__ void store(__half* p, const float* f) {
    uint4 v;
    v.x = pack_f16x2(f[0], f[1]); v.y = pack_f16x2(f[2], f[3]);
    v.z = pack_f16x2(f[4], f[5]); v.w = pack_f16x2(f[6], f[7]);
    *reinterpret_cast<uint4*>(p) = v;
  }
};
template <> struct Vec8<__nv_bfloat16> {
  static __device__ __forceinline__ void load(const __nv_bfloat16* p, float* f) {
    uint4 v = __ldg(reinterpret_cast<const uint4*>(p));
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) { float2 x = __bfloat1622float2(h[i]); f[2 * i] = x.x; f[2 * i + 1] = x.y; }
  }
  static __device__ __forceinline__ void store(__nv_bfloat16* p, const float* f) {
    uint4 v;
    v.x = pack_bf16x2(f[0], f[1]); v.y = pack_bf16x2(f[2], f[3]);
    v.z = pack_bf16x2(f[4], f[5]); v.w = pack_bf16x2(f[6], f[7]);
    *reinterpret_cast<uint4*>(p) = v;
  }
};
template <> struct Vec8<float> {
  static __device__ __forceinline__ void load(const float* p, float* f) {
    float4 a = __ldg(reinterpret_cast<const float4*>(p));
    float4 b = __ldg(reinterpret_cast<const float4*>(p) + 1);
    f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
  }
  static __device__ __forceinline__ void store(float* p, const float* f) {
    reinterpret_cast<float4*>(p)[0] = make_float4(f[0], f[1], f[2], f[3]);
    reinterpret_cast<float4*>(p)[1] = make_float4(f[4], f[5], f[6], f[7]);
  }
};

// grid (T, ceil(D / 2048)), 256 threads x 8 elements.
template <typename T>
__global__ void __launch_bounds__(256)
moe_reduce_kernel(const T* __restrict__ x, T* __restrict__ y, const uint8_t* __restrict__ mask,
                  const float* __restrict__ weights, const int* __restrict__ row_index, int topk,
                  int model_dim) {
  const int t = blockIdx.x;
  const int col = (blockIdx.y * 256 + threadIdx.x) * 8;
  if (col >= model_dim) return;
  float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  for (int s = 0; s < topk; ++s) {
    if (mask != nullptr && mask[size_t(t) * topk + s] == 0) continue;
    float f[8];
    long long row = (long long)t * topk + s;
    if (row_index != nullptr) {
      row = __ldg(row_index + row);
      if (row < 0) continue;
    }
    Vec8<T>::load(x + row * model_dim + col, f);
    const float w = weights != nullptr ? __ldg(weights + size_t(t) * topk + s) : 1.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = weights != nullptr ? fmaf(f[i], w, acc[i]) : acc[i] + f[i];
  }
  Vec8<T>::store(y + size_t(t) * model_dim + col, acc);
}

// ---------------------------------------------------------------------------- inverse
__global__ void __launch_bounds__(256)
fill_i32_kernel(int* __restrict__ p, int n, int v) {
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) p[i] = v;
}
__global__ void __launch_bounds__(256)
sorted_inverse_kernel(const int* __restrict__ sorted_ids, const int* __restrict__ num_valid_ids,
                      int* __restrict__ inverse, int num_tokens, int topk, int max_rows) {
  const int valid = min(__ldg(num_valid_ids), max_rows);
  for (int r = blockIdx.x * blockDim.x + threadIdx.x; r < valid; r += gridDim.x * blockDim.x) {
    const int id = __ldg(sorted_ids + r);
    const int t = id_token(id), s = id_slot(id);
    if (t < num_tokens && s < topk) inverse[t * topk + s] = r;
  }
}

// ---------------------------------------------------------------------------- quantiser
// One warp per (row, 128-column group): 4 elements per lane.
template <typename T>
__global__ void __launch_bounds__(256)
quant_act_1x128_kernel(const T* __restrict__ x, uint8_t* __restrict__ q, float* __restrict__ scale,
                       long long scale_stride, int rows, int groups) {
  const int lane = threadIdx.x & 31;
  const long long total = (long long)rows * groups;
  const int warps_per_block = blockDim.x >> 5;
  for (long long g = (long long)blockIdx.x * warps_per_block + (threadIdx.x >> 5); g < total;
       g += (long long)gridDim.x * warps_per_block) {
    const int r = int(g / groups), gb = int(g - (long long)r * groups);
    const T* p = x + (size_t(r) * groups + gb) * 128 + lane * 4;
    float f[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) f[i] = float(p[i]);
    float amax = fmaxf(fmaxf(fabsf(f[0]), fabsf(f[1])), fmaxf(fabsf(f[2]), fabsf(f[3])));
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
    float sc = __fdiv_rn(amax, 448.0f);
    if (sc == 0.f) sc = 1.f;
    const uint32_t packed = float4_to_e4m3x4(__fdiv_rn(f[0], sc), __fdiv_rn(f[1], sc),
                                             __fdiv_rn(f[2], sc), __fdiv_rn(f[3], sc));
    *reinterpret_cast<uint32_t*>(q + (size_t(r) * groups + gb) * 128 + lane * 4) = packed;
    if (lane == 0) scale[(long long)gb * scale_stride + r] = sc;
  }
}

// ---------------------------------------------------------------------------- shuffle
// Preshuffle order of a [rows, cols] matrix of 1- or 2-byte elements: 16 rows x 32 elements form a group,
// stored as (32 * elem_bytes / 16) 16-byte chunks of 16 rows each, i.e. element (n, k) lives in 16-byte
// vector (((n/16) * (cols/32) + k/32) * cpg + (k%32) / (16/elem_bytes)) * 16 + n%16, cpg = 2 * elem_bytes.
// One thread moves 16 bytes.
__global__ void __launch_bounds__(256)
shuffle_weight_kernel(const uint4* __restrict__ src, uint4* __restrict__ dst, long long rows, int row_bytes,
                      int cpg, int to_plain) {
  const int kv = row_bytes / 16;  // 16-byte vectors per row
  const long long nvec = rows * kv;
  const int groups = kv / cpg;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nvec;
       i += (long long)gridDim.x * blockDim.x) {
    const long long n = i / kv;
    const int kc = int(i - n * kv);              // 16-byte chunk index along k
    const long long shuf = (((n / 16) * groups + kc / cpg) * cpg + (kc % cpg)) * 16 + (n % 16);
    if (to_plain) dst[i] = __ldg(src + shuf);
    else dst[shuf] = __ldg(src + i);
  }
}

// Packed int4 weights of the reference (tests/kernels/test_moe_gemm.py:49-65 there): the signed 4-bit values
// of the 16x16-preshuffled one-byte layout, eight consecutive ones v0..v7 in four bytes b_i = (v_{i+4} << 4) | v_i.
// One thread unpacks four bytes to eight row-major values (the eight lie in one 16-byte chunk of one row).
// With gscale (bf16 output only) every value is multiplied by the scale of its 32-wide K group before it is
// rounded: scale[e][k/32][n] as f32 [E, K/32, N], or as bf16 pairs [E, K/64, N, 2] (two adjacent groups of one
// weight row in one 32-bit word: tests/utils.py:99-129 of the reference).
template <typename OutT>
__global__ void __launch_bounds__(256)
unpack_int4_weight_kernel(const uint32_t* __restrict__ packed, OutT* __restrict__ dst, long long rows, int cols,
                          const void* __restrict__ gscale, int gscale_is_bf16, int rows_per_expert) {
  const long long nquads = rows * cols / 8;
  const int groups = cols / 32;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nquads;
       i += (long long)gridDim.x * blockDim.x) {
    const uint32_t w = __ldg(packed + i);
    const long long chunk = i >> 1;                  // 16-byte chunk of the preshuffled one-byte layout
    const int off = int(i & 1) * 8;
    const int n16 = int(chunk & 15);
    long long rest = chunk >> 4;
    const int kcl = int(rest & 1);
    rest >>= 1;
    const int kg = int(rest % groups);
    const long long nb = rest / groups;
    const long long n = nb * 16 + n16;
    const int k = (kg * 2 + kcl) * 16 + off;
    float sc = 1.f;
    if (sizeof(OutT) == 2 && gscale != nullptr) {
      const long long e = n / rows_per_expert;
      const long long nl = n - e * rows_per_expert;
      if (gscale_is_bf16)
        sc = __bfloat162float(__ldg(static_cast<const __nv_bfloat16*>(gscale) +
                                    ((e * (groups / 2) + kg / 2) * rows_per_expert + nl) * 2 + (kg & 1)));
      else
        sc = __ldg(static_cast<const float*>(gscale) + (e * groups + kg) * rows_per_expert + nl);
    }
    OutT* out = dst + n * cols + k;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int b = int((w >> (8 * j)) & 0xFFu);
      const int lo = ((b & 0xF) ^ 8) - 8, hi = ((b >> 4) ^ 8) - 8;
      if constexpr (sizeof(OutT) == 1) {
        out[j] = OutT(lo);
        out[j + 4] = OutT(hi);
      } else {
        out[j] = __float2bfloat16(float(lo) * sc);
        out[j + 4] = __float2bfloat16(float(hi) * sc);
      }
    }
  }
}

}  // namespace flymoe

extern "C" int flymoe_gather_rows(const void* src, void* dst, const int32_t* sorted_ids,
                                  const int32_t* num_valid_ids, int num_tokens, int topk,
                                  int row_bytes, int src_layout, int max_rows, void* stream) {
  using namespace flymoe;
  FLYMOE_REQUIRE(src && dst && sorted_ids && num_valid_ids, "gather_rows: null pointer");
  FLYMOE_REQUIRE(row_bytes > 0 && row_bytes % 16 == 0, "gather_rows: row_bytes must be a multiple of 16");
  FLYMOE_REQUIRE(aligned16(src) && aligned16(dst), "gather_rows: pointers must be 16-byte aligned");
  FLYMOE_REQUIRE(src_layout == FLYMOE_ROWS_BY_TOKEN || src_layout == FLYMOE_ROWS_BY_PAIR ||
                     src_layout == FLYMOE_ROWS_BY_SLOT,
                 "gather_rows: src_layout must be BY_TOKEN, BY_PAIR or BY_SLOT");
  if (max_rows <= 0) return FLYMOE_OK;
  const int blocks = std::min(ceil_div(max_rows, 8), sm_count() * 8);
  gather_rows_kernel<<<blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint4*>(src), static_cast<uint4*>(dst), sorted_ids, num_valid_ids, num_tokens,
      topk, row_bytes / 16, src_layout, max_rows);
  FLYMOE_CUDA_CHECK(cudaGetLastError());
  return FLYMOE_OK;
}

extern "C" int flymoe_dispatch_rows(const void* x, const float* x_scale, const int32_t* sorted_ids,
                                    const int32_t* sorted_expert_ids, const int32_t* num_valid_ids,
                                    const int64_t* dst_x, const int64_t* dst_scale, const int64_t* pos_base,
                                    int64_t pos_limit, int num_tokens, int topk, int model_dim, int experts,
                                    int max_rows, void* stream) {
  using namespace flymoe;
  FLYMOE_REQUIRE(x && x_scale && sorted_ids && sorted_expert_ids && num_valid_ids && dst_x && dst_scale,
                 "dispatch_rows: null pointer");
  FLYMOE_REQUIRE(model_dim > 0 && model_dim % 128 == 0, "dispatch_rows: model_dim must be a positive multiple of 128");
  FLYMOE_REQUIRE(num_tokens >= 0 && topk >= 1 && experts >= 1, "dispatch_rows: bad sizes");
  FLYMOE_REQUIRE(aligned16(x), "dispatch_rows: x must be 16-byte aligned");
  if (max_rows <= 0) return FLYMOE_OK;
  int* status = device_status_ptr();
  FLYMOE_REQUIRE(status != nullptr, "dispatch_rows: no CUDA device");
  const int blocks = std::min(ceil_div(max_rows, 8), sm_count() * 4);     // 4 x 256 threads x 64 registers fit an SM
  dispatch_rows_kernel<<<blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint4*>(x), x_scale, sorted_ids, sorted_expert_ids, num_valid_ids,
      reinterpret_cast<const long long*>(dst_x), reinterpret_cast<const long long*>(dst_scale),
      reinterpret_cast<const long long*>(pos_base), static_cast<long long>(pos_limit), status, num_tokens, topk,
      model_dim / 16, model_dim / 128, experts, max_rows);
  FLYMOE_CUDA_CHECK(cudaGetLastError());
  return FLYMOE_OK;
}

extern "C" int flymoe_moe_reduce(const void* x, void* y, const uint8_t* valid_mask,
                                 const float* weights, const int32_t* row_index, int num_tokens,
                                 int topk, int model_dim, int dtype, void* stream) {
  using namespace flymoe;
  FLYMOE_REQUIRE(num_tokens >= 0 && topk >= 1 && model_dim >= 8 && model_dim % 8 == 0,
                 "moe_reduce: model_dim must be a positive multiple of 8");
  if (num_tokens == 0) return FLYMOE_OK;
  FLYMOE_REQUIRE(x && y, "moe_reduce: null pointer");
  FLYMOE_REQUIRE(aligned16(x) && aligned16(y), "moe_reduce: pointers must be 16-byte aligned");
  dim3 grid(num_tokens, ceil_div(model_dim, 2048));
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  switch (dtype) {
    case FLYMOE_F16:
      moe_reduce_kernel<__half><<<grid, 256, 0, s>>>(static_cast<const __half*>(x), static_cast<__half*>(y),
                                                     valid_mask, weights, row_index, topk, model_dim);
      break;
    case FLYMOE_BF16:
      moe_reduce_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>(static_cast<const __nv_bfloat16*>(x),
                                                            static_cast<__nv_bfloat16*>(y), valid_mask,
                                                            weights, row_index, topk, model_dim);
      break;
    case FLYMOE_F32:
      moe_reduce_kernel<float><<<grid, 256, 0, s>>>(static_cast<const float*>(x), static_cast<float*>(y),
                                                    valid_mask, weights, row_index, topk, model_dim);
      break;
    default:
      set_last_error_msg("moe_reduce: dtype must be F16, BF16 or F32");
      return FLYMOE_ERR_INVALID_ARGUMENT;
  }
  FLYMOE_CUDA_CHECK(cudaGetLastError());
  return FLYMOE_OK;
}

extern "C" int flymoe_sorted_inverse(const int32_t* sorted_ids, const int32_t* num_valid_ids,
                                     int32_t* inverse, int num_tokens, int topk, int max_rows,
                                     void* stream) {
  using namespace flymoe;
  FLYMOE_REQUIRE(num_tokens >= 0 && topk >= 1 && max_rows >= 0, "sorted_inverse: bad sizes");
  const int pairs = num_tokens * topk;
  if (pairs == 0) return FLYMOE_OK;
  FLYMOE_REQUIRE(sorted_ids && num_valid_ids && inverse, "sorted_inverse: null pointer");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  fill_i32_kernel<<<std::min(ceil_div(pairs, 256), sm_count() * 8), 256, 0, s>>>(inverse, pairs, -1);
  FLYMOE_CUDA_CHECK(cudaGetLastError());
  if (max_rows > 0) {
    sorted_inverse_kernel<<<std::min(ceil_div(max_rows, 256), sm_count() * 8), 256, 0, s>>>(
        sorted_ids, num_valid_ids, inverse, num_tokens, topk, max_rows);
    FLYMOE_CUDA_CHECK(cudaGetLastError());
  }
  return FLYMOE_OK;
}

extern "C" int flymoe_quant_act_1x128(const void* x, int x_dtype, void* q, float* scale,
                                      int64_t scale_stride, int rows, int cols, void* stream) {
  using namespace flymoe;
  FLYMOE_REQUIRE(rows >= 0 && cols > 0 && cols % 128 == 0, "quant_act_1x128: cols must be a multiple of 128");
  if (rows == 0) return FLYMOE_OK;
  FLYMOE_REQUIRE(x && q && scale, "quant_act_1x128: null pointer");
  FLYMOE_REQUIRE(scale_stride >= rows, "quant_act_1x128: scale_stride < rows");
  const int groups = cols / 128;
  const long long total = (long long)rows * groups;
  const int blocks = int(std::min<long long>((total + 7) / 8, (long long)sm_count() * 16));
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  uint8_t* qq = static_cast<uint8_t*>(q);
  switch (x_dtype) {
    case FLYMOE_F16:
      quant_act_1x128_kernel<__half><<<blocks, 256, 0, s>>>(static_cast<const __half*>(x), qq, scale,
                                                            scale_stride, rows, groups);
      break;
    case FLYMOE_BF16:
      quant_act_1x128_kernel<__nv_bfloat16><<<blocks, 256, 0, s>>>(static_cast<const __nv_bfloat16*>(x), qq,
                                                                   scale, scale_stride, rows, groups);
      break;
    case FLYMOE_F32:
      quant_act_1x128_kernel<float><<<blocks, 256, 0, s>>>(static_cast<const float*>(x), qq, scale,
                                                           scale_stride, rows, groups);
      break;
    default:
      set_last_error_msg("quant_act_1x128: dtype must be F16, BF16 or F32");
      return FLYMOE_ERR_INVALID_ARGUMENT;
  }
  FLYMOE_CUDA_CHECK(cudaGetLastError());
  return FLYMOE_OK;
}

extern "C" int flymoe_shuffle_weight_elems(const void* src, void* dst, int64_t rows, int cols, int elem_bytes,
                                           int to_plain, void* stream) {
  using namespace flymoe;
  FLYMOE_REQUIRE(src && dst && src != dst, "shuffle_weight: src and dst must be distinct non-null pointers");
  FLYMOE_REQUIRE(elem_bytes == 1 || elem_bytes == 2, "shuffle_weight: elem_bytes must be 1 or 2");
  FLYMOE_REQUIRE(rows > 0 && rows % 16 == 0 && cols > 0 && cols % 32 == 0,
                 "shuffle_weight: rows must be a multiple of 16 and cols of 32");
  FLYMOE_REQUIRE(aligned16(src) && aligned16(dst), "shuffle_weight: pointers must be 16-byte aligned");
  const int row_bytes = cols * elem_bytes;
  const long long nvec = rows * (row_bytes / 16);
  const int blocks = int(std::min<long long>((nvec + 255) / 256, (long long)sm_count() * 32));
  shuffle_weight_kernel<<<blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint4*>(src), static_cast<uint4*>(dst), rows, row_bytes, 2 * elem_bytes, to_plain);
  FLYMOE_CUDA_CHECK(cudaGetLastError());
  return FLYMOE_OK;
}

extern "C" int flymoe_shuffle_weight(const void* src, void* dst, int64_t rows, int cols, int to_plain,
                                     void* stream) {
  return flymoe_shuffle_weight_elems(src, dst, rows, cols, 1, to_plain, stream);
}

extern "C" int flymoe_unpack_int4_weight_grouped(const void* packed, void* dst, int64_t rows, int cols, int out_dtype,
                                                 const void* group_scale, int group_scale_dtype, int group_size,
                                                 int rows_per_expert, void* stream) {
  using namespace flymoe;
  FLYMOE_REQUIRE(packed && dst && packed != dst, "unpack_int4_weight: packed and dst must be distinct non-null pointers");
  FLYMOE_REQUIRE(rows > 0 && rows % 16 == 0 && cols > 0 && cols % 32 == 0,
                 "unpack_int4_weight: rows must be a multiple of 16 and cols of 32");
  FLYMOE_REQUIRE(out_dtype == FLYMOE_I8 || out_dtype == FLYMOE_BF16, "unpack_int4_weight: out_dtype must be I8 or BF16");
  FLYMOE_REQUIRE(aligned16(packed) && aligned16(dst), "unpack_int4_weight: pointers must be 16-byte aligned");
  if (group_scale != nullptr) {
    FLYMOE_REQUIRE(out_dtype == FLYMOE_BF16, "unpack_int4_weight: group scales need BF16 output");
    FLYMOE_REQUIRE(group_size == 32, "unpack_int4_weight: group_size must be 32");
    FLYMOE_REQUIRE(group_scale_dtype == FLYMOE_F32 || group_scale_dtype == FLYMOE_BF16,
                   "unpack_int4_weight: group scales must be F32 or BF16");
    FLYMOE_REQUIRE(rows_per_expert > 0 && rows % rows_per_expert == 0,
                   "unpack_int4_weight: rows must be a multiple of rows_per_expert");
    FLYMOE_REQUIRE(group_scale_dtype != FLYMOE_BF16 || cols % 64 == 0,
                   "unpack_int4_weight: bf16 group scales come in pairs, cols must be a multiple of 64");
  }
  const long long nquads = rows * cols / 8;
  const int blocks = int(std::min<long long>((nquads + 255) / 256, (long long)sm_count() * 32));
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int sbf = group_scale_dtype == FLYMOE_BF16 ? 1 : 0;
  if (out_dtype == FLYMOE_I8)
    unpack_int4_weight_kernel<int8_t><<<blocks, 256, 0, s>>>(static_cast<const uint32_t*>(packed),
                                                           static_cast<int8_t*>(dst), rows, cols, nullptr, 0, 1);
  else
    unpack_int4_weight_kernel<__nv_bfloat16><<<blocks, 256, 0, s>>>(
        static_cast<const uint32_t*>(packed), static_cast<__nv_bfloat16*>(dst), rows, cols, group_scale, sbf,
        group_scale ? rows_per_expert : 1);
  FLYMOE_CUDA_CHECK(cudaGetLastError());
  return FLYMOE_OK;
}

extern "C" int flymoe_unpack_int4_weight(const void* packed, void* dst, int64_t rows, int cols, int out_dtype,
                                         void* stream) {
  return flymoe_unpack_int4_weight_grouped(packed, dst, rows, cols, out_dtype, nullptr, 0, 0, 0, stream);
}
