// Plain CUDA-core implementation of the two grouped FP8 GEMM stages.  It follows the
// same data contract and block-scale arithmetic as the tensor-core kernels and exists
// to cross-check them on the GPU at sizes the CPU oracle cannot reach; it reads rows
// through the sorted-id list directly, so it needs no gathered copy of the activations.
#include "common.cuh"
#include "gemm_args.cuh"

namespace flymoe {

constexpr int kSimtRows = 8;      // sorted rows processed per pass
constexpr int kSimtCols = 128;    // output columns per block (= threads)

__device__ __forceinline__ void cvt16(const uint4& v, float* f, bool int8_ops) {
  const uint8_t* b = reinterpret_cast<const uint8_t*>(&v);
#pragma unroll
  for (int i = 0; i < 16; ++i) f[i] = int8_ops ? float(int(static_cast<int8_t>(b[i]))) : fp8_e4m3_to_float(b[i]);
}

__device__ __forceinline__ long long src_row(int layout, int r, int t, int s, int topk, int num_tokens) {
  if (layout == FLYMOE_ROWS_BY_TOKEN) return t;
  if (layout == FLYMOE_ROWS_BY_PAIR) return (long long)t * topk + s;
  if (layout == FLYMOE_ROWS_BY_SLOT) return (long long)s * num_tokens + t;
  return r;
}

// STAGE 1: NACC = 2 (gate, up).  STAGE 2: NACC = 1.
template <int STAGE>
__global__ void __launch_bounds__(kSimtCols)
moe_gemm_simt_kernel(GemmArgs a) {
  constexpr int NACC = STAGE == 1 ? 2 : 1;
  extern __shared__ __align__(16) uint8_t smem_raw[];
  uint8_t* xs = smem_raw;                                      // [kSimtRows][K]
  __shared__ float red[kSimtRows][4];
  const int K = a.k_dim;
  const int KB = K / 128;
  const int tid = threadIdx.x;
  const int mb = blockIdx.y;
  const int nt = blockIdx.x;
  const int valid_rows = min(__ldg(a.num_valid_ids), a.size_expert_ids * a.tile_m);
  if (mb * a.tile_m >= valid_rows) return;
  const int e = __ldg(a.sorted_expert_ids + mb);
  if (e < 0 || e >= a.experts) return;

  const int col = nt * kSimtCols + tid;                        // output column
  const int n_total = a.n_dim;                                 // stage 1: inter_dim, stage 2: model_dim
  const bool col_ok = col < n_total;
  // weight rows for this thread
  const long long wrows_per_expert = STAGE == 1 ? 2LL * a.n_dim : a.n_dim;
  const uint8_t* w0 = a.w + ((long long)e * wrows_per_expert + (col_ok ? col : 0)) * K;
  const uint8_t* w1 = STAGE == 1 ? w0 + (long long)a.n_dim * K : w0;
  const int nblk_per_expert = int(wrows_per_expert / 128);
  const bool per_token = a.scaling == FLYMOE_SCALE_PER_TOKEN;   // one scale per activation row / weight row
  const bool int8_ops = a.in_dtype == FLYMOE_I8;
  const float* sw0 = a.scale_w + ((long long)e * nblk_per_expert + (col_ok ? col : 0) / 128) * KB;
  const float* sw1 = STAGE == 1 ? sw0 + (long long)(a.n_dim / 128) * KB : sw0;
  const float* swr = a.scale_w + (long long)e * wrows_per_expert + (col_ok ? col : 0);   // per-row weight scales

  for (int rb = 0; rb < a.tile_m; rb += kSimtRows) {
    int rt[kSimtRows], rs[kSimtRows];
    bool rok[kSimtRows];
    long long srow[kSimtRows], sidx[kSimtRows];
#pragma unroll
    for (int i = 0; i < kSimtRows; ++i) {
      const int r = mb * a.tile_m + rb + i;
      rok[i] = false; rt[i] = 0; rs[i] = 0; srow[i] = 0; sidx[i] = 0;
      if (rb + i < a.tile_m && r < valid_rows) {
        const int id = __ldg(a.sorted_ids + r);
        rt[i] = id_token(id); rs[i] = id_slot(id);
        rok[i] = rt[i] < a.num_tokens && rs[i] < a.topk;
        if (rok[i]) {
          srow[i] = src_row(a.a_layout, r, rt[i], rs[i], a.topk, a.num_tokens);
          sidx[i] = src_row(a.a_scale_layout, r, rt[i], rs[i], a.topk, a.num_tokens);
        }
      }
    }
    __syncthreads();
#pragma unroll
    for (int i = 0; i < kSimtRows; ++i) {
      uint4* d = reinterpret_cast<uint4*>(xs + size_t(i) * K);
      if (rok[i]) {
        const uint4* p = reinterpret_cast<const uint4*>(a.a + srow[i] * K);
        for (int v = tid; v < K / 16; v += kSimtCols) d[v] = __ldg(p + v);
      } else {
        for (int v = tid; v < K / 16; v += kSimtCols) d[v] = make_uint4(0, 0, 0, 0);
      }
    }
    __syncthreads();

    float acc[NACC][kSimtRows];
#pragma unroll
    for (int j = 0; j < NACC; ++j)
#pragma unroll
      for (int i = 0; i < kSimtRows; ++i) acc[j][i] = 0.f;

    if (col_ok) {
      for (int kb = 0; kb < KB; ++kb) {
        float part[NACC][kSimtRows];
#pragma unroll
        for (int j = 0; j < NACC; ++j)
#pragma unroll
          for (int i = 0; i < kSimtRows; ++i) part[j][i] = 0.f;
        for (int kc = 0; kc < 8; ++kc) {
          const int koff = kb * 128 + kc * 16;
          float wf[NACC][16];
          cvt16(__ldg(reinterpret_cast<const uint4*>(w0 + koff)), wf[0], int8_ops);
          if (NACC == 2) cvt16(__ldg(reinterpret_cast<const uint4*>(w1 + koff)), wf[NACC - 1], int8_ops);
#pragma unroll
          for (int i = 0; i < kSimtRows; ++i) {
            float xf[16];
            cvt16(*reinterpret_cast<const uint4*>(xs + size_t(i) * K + koff), xf, int8_ops);
#pragma unroll
            for (int j = 0; j < NACC; ++j)
#pragma unroll
              for (int q = 0; q < 16; ++q) part[j][i] = fmaf(xf[q], wf[j][q], part[j][i]);
          }
        }
        const float s0 = per_token ? 1.f : __ldg(sw0 + kb);
        const float s1 = per_token ? 1.f : __ldg(sw1 + kb);
#pragma unroll
        for (int i = 0; i < kSimtRows; ++i) {
          const float sa = !rok[i] ? 0.f : per_token ? 1.f
                         : __ldg(a.scale_a + (long long)kb * a.sa_stride + sidx[i] * a.sa_row_stride);
          acc[0][i] = fmaf(part[0][i], sa * s0, acc[0][i]);
          if (NACC == 2) acc[NACC - 1][i] = fmaf(part[NACC - 1][i], sa * s1, acc[NACC - 1][i]);
        }
      }
      if (per_token) {
        const float c0 = __ldg(swr);
        const float c1 = STAGE == 1 ? __ldg(swr + a.n_dim) : c0;
#pragma unroll
        for (int i = 0; i < kSimtRows; ++i) {
          const float sa = rok[i] ? __ldg(a.scale_a + sidx[i]) : 0.f;
          acc[0][i] *= sa * c0;
          if (NACC == 2) acc[NACC - 1][i] *= sa * c1;
        }
      }
    }

    // ---- epilogue -----------------------------------------------------------------
#pragma unroll
    for (int i = 0; i < kSimtRows; ++i) {
      const int r = mb * a.tile_m + rb + i;
      const bool in_tile = (rb + i < a.tile_m) && r < valid_rows;   // block-uniform
      if (!in_tile) continue;
      const float wgt = (a.doweight && rok[i]) ? __ldg(a.sorted_weights + r) : 1.f;
      if (STAGE == 1) {
        float h = rok[i] ? silu_f32(acc[0][i]) * acc[NACC - 1][i] * wgt : 0.f;
        const long long orow = (a.out_layout == FLYMOE_ROWS_SORTED) ? r : (long long)rt[i] * a.topk + rs[i];
        if (a.out_dtype == FLYMOE_E4M3) {
          // amax over the 128 columns of this block (= one quantisation group)
          float m = col_ok ? fabsf(h) : 0.f;
#pragma unroll
          for (int off = 16; off > 0; off >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, off));
          if ((tid & 31) == 0) red[i][tid >> 5] = m;
          __syncthreads();
          m = fmaxf(fmaxf(red[i][0], red[i][1]), fmaxf(red[i][2], red[i][3]));
          float sc = __fdiv_rn(m, 448.0f);
          if (sc == 0.f) sc = 1.f;
          const bool wr = rok[i] || a.out_layout == FLYMOE_ROWS_SORTED;   // pad rows: zeros in sorted layout
          if (wr && col_ok) {
            const uint16_t c2 = float2_to_e4m3x2(__fdiv_rn(h, sc), 0.f);
            static_cast<uint8_t*>(a.out)[orow * n_total + col] = uint8_t(c2 & 0xFF);
            if (tid == 0) a.out_scale[(long long)nt * a.out_scale_stride + orow] = sc;
          }
        } else if (rok[i] && col_ok) {
          if (a.out_dtype == FLYMOE_F16) static_cast<__half*>(a.out)[orow * n_total + col] = __float2half_rn(h);
          else static_cast<__nv_bfloat16*>(a.out)[orow * n_total + col] = __float2bfloat16_rn(h);
        }
      } else {
        if (!rok[i] || !col_ok) continue;
        const float v = acc[0][i] * wgt;
        if (a.accumulate) {
          const long long o = (long long)rt[i] * n_total + col;
          if (a.out_dtype == FLYMOE_F32) atomicAdd(static_cast<float*>(a.out) + o, v);
          else if (a.out_dtype == FLYMOE_F16) atomicAdd(static_cast<__half*>(a.out) + o, __float2half_rn(v));
          else atomicAdd(static_cast<__nv_bfloat16*>(a.out) + o, __float2bfloat16_rn(v));
        } else {
          const long long o = ((long long)rt[i] * a.topk + rs[i]) * n_total + col;
          if (a.out_dtype == FLYMOE_F16) static_cast<__half*>(a.out)[o] = __float2half_rn(v);
          else static_cast<__nv_bfloat16*>(a.out)[o] = __float2bfloat16_rn(v);
        }
      }
    }
  }
}

int launch_gemm_simt(int stage, const GemmArgs& a, cudaStream_t stream) {
  dim3 grid(ceil_div(a.n_dim, kSimtCols), a.size_expert_ids);
  const size_t smem = size_t(kSimtRows) * a.k_dim;
  if (stage == 1) {
    if (smem > 48 * 1024)
      FLYMOE_CUDA_CHECK(cudaFuncSetAttribute(moe_gemm_simt_kernel<1>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)));
    moe_gemm_simt_kernel<1><<<grid, kSimtCols, smem, stream>>>(a);
  } else {
    if (smem > 48 * 1024)
      FLYMOE_CUDA_CHECK(cudaFuncSetAttribute(moe_gemm_simt_kernel<2>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)));
    moe_gemm_simt_kernel<2><<<grid, kSimtCols, smem, stream>>>(a);
  }
  FLYMOE_CUDA_CHECK(cudaGetLastError());
  return FLYMOE_OK;
}

}  // namespace flymoe
