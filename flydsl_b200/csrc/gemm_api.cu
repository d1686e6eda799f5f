// C entry points of the two grouped-GEMM stages: argument validation and dispatch.
#include "common.cuh"
#include "gemm_args.cuh"

using namespace flymoe;

static bool layout_ok(int l) {
  return l == FLYMOE_ROWS_BY_TOKEN || l == FLYMOE_ROWS_BY_PAIR || l == FLYMOE_ROWS_SORTED || l == FLYMOE_ROWS_BY_SLOT;
}

static bool is_half(int dtype) { return dtype == FLYMOE_F16 || dtype == FLYMOE_BF16; }

static long long layout_rows(int layout, int num_tokens, int topk, int size_expert_ids, int tile_m) {
  if (layout == FLYMOE_ROWS_BY_TOKEN) return num_tokens;
  if (layout == FLYMOE_ROWS_BY_PAIR || layout == FLYMOE_ROWS_BY_SLOT) return (long long)num_tokens * topk;
  return (long long)size_expert_ids * tile_m;
}

static int gemm1_impl(void* out, float* out_scale, int64_t out_scale_stride, const void* x, const float* scale_x,
                      int64_t sx_stride, int64_t sx_row_stride, const void* w, const float* scale_w,
                      const int32_t* sorted_ids, const int32_t* sorted_expert_ids, const float* sorted_weights,
                      const int32_t* num_valid_ids, int num_tokens, int inter_dim, int model_dim,
                      int size_expert_ids, int experts, int topk, int tile_m, int doweight, int out_dtype,
                      int x_layout, int x_scale_layout, int out_layout, int impl, int scaling, int in_dtype,
                      void* stream) {
  const bool per_token = scaling == FLYMOE_SCALE_PER_TOKEN;
  FLYMOE_REQUIRE(num_tokens >= 0 && num_tokens < (1 << 24), "gemm1: num_tokens out of range");
  FLYMOE_REQUIRE(inter_dim > 0 && inter_dim % 128 == 0, "gemm1: inter_dim must be a positive multiple of 128");
  FLYMOE_REQUIRE(model_dim > 0 && model_dim % 128 == 0, "gemm1: model_dim must be a positive multiple of 128");
  FLYMOE_REQUIRE(experts >= 1 && topk >= 1 && topk <= 255, "gemm1: experts/topk out of range");
  FLYMOE_REQUIRE(tile_m >= 1 && size_expert_ids >= 0, "gemm1: tile_m/size_expert_ids out of range");
  // F32 with per-token scaling: the raw gate|up sums of the reference's split-K contract, [T*k, 2I], added to out
  const bool raw_sums = out_dtype == FLYMOE_F32 && per_token;
  FLYMOE_REQUIRE(out_dtype == FLYMOE_F16 || out_dtype == FLYMOE_BF16 || (out_dtype == FLYMOE_E4M3 && !per_token) || raw_sums,
                 "gemm1: out_dtype must be F16, BF16, (block-scaled only) E4M3 or (per-token only) F32");
  FLYMOE_REQUIRE(!raw_sums || (impl == FLYMOE_IMPL_TCGEN05 && out_layout == FLYMOE_ROWS_BY_PAIR),
                 "gemm1: fp32 gate|up sums need the tcgen05 kernel and out_layout BY_PAIR");
  FLYMOE_REQUIRE(in_dtype == FLYMOE_E4M3 || ((in_dtype == FLYMOE_I8 || is_half(in_dtype)) && per_token),
                 "gemm1: in_dtype must be E4M3 or (per-token scaling only) I8, F16, BF16");
  FLYMOE_REQUIRE(!is_half(in_dtype) || impl == FLYMOE_IMPL_TCGEN05, "gemm1: 16-bit operands need the tcgen05 kernel");
  const bool x_per_pair = x_layout == FLYMOE_ROWS_BY_PAIR || x_layout == FLYMOE_ROWS_BY_SLOT;
  const bool sx_per_pair = x_scale_layout == FLYMOE_ROWS_BY_PAIR || x_scale_layout == FLYMOE_ROWS_BY_SLOT;
  FLYMOE_REQUIRE(layout_ok(x_layout) && (!x_per_pair || per_token),
                 "gemm1: x_layout must be BY_TOKEN or SORTED (BY_PAIR / BY_SLOT with per-token scaling)");
  FLYMOE_REQUIRE(layout_ok(x_scale_layout) && (!sx_per_pair || per_token),
                 "gemm1: x_scale_layout must be BY_TOKEN or SORTED (BY_PAIR / BY_SLOT with per-token scaling)");
  FLYMOE_REQUIRE(out_layout == FLYMOE_ROWS_BY_PAIR || out_layout == FLYMOE_ROWS_SORTED,
                 "gemm1: out_layout must be BY_PAIR or SORTED");
  if (num_tokens == 0 || size_expert_ids == 0) return FLYMOE_OK;
  FLYMOE_REQUIRE(out && x && w && sorted_ids && sorted_expert_ids && num_valid_ids, "gemm1: null pointer");
  FLYMOE_REQUIRE((scale_x && scale_w) || is_half(in_dtype), "gemm1: scales may be null only with 16-bit operands");
  FLYMOE_REQUIRE(!doweight || sorted_weights, "gemm1: doweight needs sorted_weights");
  FLYMOE_REQUIRE(out_dtype != FLYMOE_E4M3 || out_scale, "gemm1: e4m3 output needs out_scale");
  FLYMOE_REQUIRE(aligned16(out) && aligned16(x) && aligned16(w), "gemm1: out/x/w must be 16-byte aligned");
  FLYMOE_REQUIRE(!per_token || aligned16(scale_w), "gemm1: per-row weight scales must be 16-byte aligned");
  const long long srows = layout_rows(x_scale_layout, num_tokens, topk, size_expert_ids, tile_m);
  FLYMOE_REQUIRE(sx_row_stride >= 1 && sx_stride >= 1, "gemm1: scale strides must be positive");
  FLYMOE_REQUIRE(per_token || sx_row_stride != 1 || sx_stride >= srows || x_scale_layout == FLYMOE_ROWS_SORTED,
                 "gemm1: sx_stride smaller than row count");
  int* status = device_status_ptr();
  FLYMOE_REQUIRE(status != nullptr, "gemm1: no CUDA device");

  GemmArgs a;
  a.a = static_cast<const uint8_t*>(x);
  a.scale_a = scale_x;
  a.sa_stride = sx_stride;
  a.sa_row_stride = sx_row_stride;
  a.a_layout = x_layout;
  a.a_scale_layout = x_scale_layout;
  a.a_rows = layout_rows(x_layout, num_tokens, topk, size_expert_ids, tile_m);
  a.w = static_cast<const uint8_t*>(w);
  a.scale_w = scale_w;
  a.sorted_ids = sorted_ids;
  a.sorted_expert_ids = sorted_expert_ids;
  a.sorted_weights = sorted_weights;
  a.num_valid_ids = num_valid_ids;
  a.out = out;
  a.out_scale = out_scale;
  a.out_scale_stride = out_scale_stride;
  a.out_dtype = out_dtype;
  a.out_layout = out_layout;
  a.accumulate = 0;
  a.row_dst = nullptr;
  a.doweight = doweight;
  a.scaling = scaling;
  a.in_dtype = in_dtype;
  a.num_tokens = num_tokens;
  a.topk = topk;
  a.experts = experts;
  a.n_dim = inter_dim;
  a.k_dim = is_half(in_dtype) ? 2 * model_dim : model_dim;      // the kernels count K in bytes
  a.size_expert_ids = size_expert_ids;
  a.tile_m = tile_m;
  a.status = status;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (impl == FLYMOE_IMPL_SIMT) return launch_gemm_simt(1, a, s);
  if (impl == FLYMOE_IMPL_TCGEN05) return launch_gemm_sm100(1, a, s);
  set_last_error_msg("gemm1: unknown impl");
  return FLYMOE_ERR_INVALID_ARGUMENT;
}

extern "C" int flymoe_moe_gemm1(void* out, float* out_scale, int64_t out_scale_stride, const void* x,
                                const float* scale_x, int64_t sx_stride, int64_t sx_row_stride, const void* w,
                                const float* scale_w, const int32_t* sorted_ids,
                                const int32_t* sorted_expert_ids, const float* sorted_weights,
                                const int32_t* num_valid_ids, int num_tokens, int inter_dim,
                                int model_dim, int size_expert_ids, int experts, int topk, int tile_m,
                                int doweight, int out_dtype, int x_layout, int x_scale_layout,
                                int out_layout, int impl, void* stream) {
  return gemm1_impl(out, out_scale, out_scale_stride, x, scale_x, sx_stride, sx_row_stride, w, scale_w, sorted_ids,
                    sorted_expert_ids, sorted_weights, num_valid_ids, num_tokens, inter_dim, model_dim,
                    size_expert_ids, experts, topk, tile_m, doweight, out_dtype, x_layout, x_scale_layout,
                    out_layout, impl, FLYMOE_SCALE_BLOCK128, FLYMOE_E4M3, stream);
}

extern "C" int flymoe_moe_gemm1_pertoken(void* out, const void* x, const float* scale_x, const void* w,
                                         const float* scale_w, const int32_t* sorted_ids,
                                         const int32_t* sorted_expert_ids, const float* sorted_weights,
                                         const int32_t* num_valid_ids, int num_tokens, int inter_dim,
                                         int model_dim, int size_expert_ids, int experts, int topk, int tile_m,
                                         int doweight, int in_dtype, int out_dtype, int x_layout,
                                         int x_scale_layout, int out_layout, int impl, void* stream) {
  return gemm1_impl(out, nullptr, 0, x, scale_x, 1, 1, w, scale_w, sorted_ids, sorted_expert_ids, sorted_weights,
                    num_valid_ids, num_tokens, inter_dim, model_dim, size_expert_ids, experts, topk, tile_m, doweight,
                    out_dtype, x_layout, x_scale_layout, out_layout, impl, FLYMOE_SCALE_PER_TOKEN, in_dtype, stream);
}

static int gemm2_impl(void* out, const unsigned long long* row_dst, const void* a2, const float* scale_a,
                      int64_t sa_stride, const void* w, const float* scale_w, const int32_t* sorted_ids,
                      const int32_t* sorted_expert_ids, const float* sorted_weights,
                      const int32_t* num_valid_ids, int num_tokens, int model_dim,
                      int inter_dim, int size_expert_ids, int experts, int topk, int tile_m,
                      int doweight, int out_dtype, int accumulate, int a_layout,
                      int a_scale_layout, int impl, int scaling, int in_dtype, void* stream) {
  const bool per_token = scaling == FLYMOE_SCALE_PER_TOKEN;
  FLYMOE_REQUIRE(num_tokens >= 0 && num_tokens < (1 << 24), "gemm2: num_tokens out of range");
  FLYMOE_REQUIRE(inter_dim > 0 && inter_dim % 128 == 0, "gemm2: inter_dim must be a positive multiple of 128");
  FLYMOE_REQUIRE(model_dim > 0 && model_dim % 128 == 0, "gemm2: model_dim must be a positive multiple of 128");
  FLYMOE_REQUIRE(experts >= 1 && topk >= 1 && topk <= 255, "gemm2: experts/topk out of range");
  FLYMOE_REQUIRE(tile_m >= 1 && size_expert_ids >= 0, "gemm2: tile_m/size_expert_ids out of range");
  FLYMOE_REQUIRE(out_dtype == FLYMOE_F16 || out_dtype == FLYMOE_BF16 || (out_dtype == FLYMOE_F32 && accumulate),
                 "gemm2: out_dtype must be F16 or BF16 (F32 only with accumulate)");
  FLYMOE_REQUIRE(in_dtype == FLYMOE_E4M3 || ((in_dtype == FLYMOE_I8 || is_half(in_dtype)) && per_token),
                 "gemm2: in_dtype must be E4M3 or (per-token scaling only) I8, F16, BF16");
  FLYMOE_REQUIRE(!is_half(in_dtype) || impl == FLYMOE_IMPL_TCGEN05, "gemm2: 16-bit operands need the tcgen05 kernel");
  FLYMOE_REQUIRE((a_layout == FLYMOE_ROWS_BY_PAIR || a_layout == FLYMOE_ROWS_SORTED) &&
                     (a_scale_layout == FLYMOE_ROWS_BY_PAIR || a_scale_layout == FLYMOE_ROWS_SORTED),
                 "gemm2: a_layout/a_scale_layout must be BY_PAIR or SORTED");
  if (num_tokens == 0 || size_expert_ids == 0) return FLYMOE_OK;
  FLYMOE_REQUIRE((out || row_dst) && a2 && w && sorted_ids && sorted_expert_ids && num_valid_ids, "gemm2: null pointer");
  FLYMOE_REQUIRE((scale_a && scale_w) || is_half(in_dtype), "gemm2: scales may be null only with 16-bit operands");
  FLYMOE_REQUIRE(!row_dst || (!accumulate && out_dtype != FLYMOE_F32 && impl == FLYMOE_IMPL_TCGEN05 && !per_token),
                 "gemm2: per-row destinations need accumulate == 0, a 16-bit out_dtype and the block-scaled tcgen05 kernel");
  FLYMOE_REQUIRE(!doweight || sorted_weights, "gemm2: doweight needs sorted_weights");
  FLYMOE_REQUIRE(aligned16(out) && aligned16(a2) && aligned16(w), "gemm2: out/a2/w must be 16-byte aligned");
  FLYMOE_REQUIRE(!per_token || aligned16(scale_w), "gemm2: per-row weight scales must be 16-byte aligned");
  int* status = device_status_ptr();
  FLYMOE_REQUIRE(status != nullptr, "gemm2: no CUDA device");

  GemmArgs a;
  a.a = static_cast<const uint8_t*>(a2);
  a.scale_a = scale_a;
  a.sa_stride = sa_stride;
  a.sa_row_stride = 1;
  a.a_layout = a_layout;
  a.a_scale_layout = a_scale_layout;
  a.a_rows = layout_rows(a_layout, num_tokens, topk, size_expert_ids, tile_m);
  a.w = static_cast<const uint8_t*>(w);
  a.scale_w = scale_w;
  a.sorted_ids = sorted_ids;
  a.sorted_expert_ids = sorted_expert_ids;
  a.sorted_weights = sorted_weights;
  a.num_valid_ids = num_valid_ids;
  a.out = out;
  a.out_scale = nullptr;
  a.out_scale_stride = 0;
  a.out_dtype = out_dtype;
  a.out_layout = FLYMOE_ROWS_BY_PAIR;
  a.accumulate = accumulate ? 1 : 0;
  a.row_dst = row_dst;
  a.doweight = doweight;
  a.scaling = scaling;
  a.in_dtype = in_dtype;
  a.num_tokens = num_tokens;
  a.topk = topk;
  a.experts = experts;
  a.n_dim = model_dim;
  a.k_dim = is_half(in_dtype) ? 2 * inter_dim : inter_dim;
  a.size_expert_ids = size_expert_ids;
  a.tile_m = tile_m;
  a.status = status;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (impl == FLYMOE_IMPL_SIMT) return launch_gemm_simt(2, a, s);
  if (impl == FLYMOE_IMPL_TCGEN05) return launch_gemm_sm100(2, a, s);
  set_last_error_msg("gemm2: unknown impl");
  return FLYMOE_ERR_INVALID_ARGUMENT;
}

extern "C" int flymoe_moe_gemm2(void* out, const void* a2, const float* scale_a, int64_t sa_stride,
                                const void* w, const float* scale_w, const int32_t* sorted_ids,
                                const int32_t* sorted_expert_ids, const float* sorted_weights,
                                const int32_t* num_valid_ids, int num_tokens, int model_dim,
                                int inter_dim, int size_expert_ids, int experts, int topk, int tile_m,
                                int doweight, int out_dtype, int accumulate, int a_layout,
                                int a_scale_layout, int impl, void* stream) {
  return gemm2_impl(out, nullptr, a2, scale_a, sa_stride, w, scale_w, sorted_ids, sorted_expert_ids, sorted_weights,
                    num_valid_ids, num_tokens, model_dim, inter_dim, size_expert_ids, experts, topk, tile_m, doweight,
                    out_dtype, accumulate, a_layout, a_scale_layout, impl, FLYMOE_SCALE_BLOCK128, FLYMOE_E4M3, stream);
}

extern "C" int flymoe_moe_gemm2_pertoken(void* out, const void* a2, const float* scale_a, const void* w,
                                         const float* scale_w, const int32_t* sorted_ids,
                                         const int32_t* sorted_expert_ids, const float* sorted_weights,
                                         const int32_t* num_valid_ids, int num_tokens, int model_dim,
                                         int inter_dim, int size_expert_ids, int experts, int topk, int tile_m,
                                         int doweight, int in_dtype, int out_dtype, int accumulate, int a_layout,
                                         int a_scale_layout, int impl, void* stream) {
  return gemm2_impl(out, nullptr, a2, scale_a, 1, w, scale_w, sorted_ids, sorted_expert_ids, sorted_weights,
                    num_valid_ids, num_tokens, model_dim, inter_dim, size_expert_ids, experts, topk, tile_m, doweight,
                    out_dtype, accumulate, a_layout, a_scale_layout, impl, FLYMOE_SCALE_PER_TOKEN, in_dtype, stream);
}

extern "C" int flymoe_moe_gemm2_scatter_rows(const uint64_t* row_dst, const void* a2, const float* scale_a,
                                             int64_t sa_stride, const void* w, const float* scale_w,
                                             const int32_t* sorted_ids, const int32_t* sorted_expert_ids,
                                             const float* sorted_weights, const int32_t* num_valid_ids,
                                             int num_tokens, int model_dim, int inter_dim, int size_expert_ids,
                                             int experts, int topk, int tile_m, int doweight, int out_dtype,
                                             int a_layout, int a_scale_layout, void* stream) {
  FLYMOE_REQUIRE(row_dst != nullptr, "gemm2_scatter_rows: row_dst is null");
  return gemm2_impl(nullptr, reinterpret_cast<const unsigned long long*>(row_dst), a2, scale_a, sa_stride, w, scale_w,
                    sorted_ids, sorted_expert_ids, sorted_weights, num_valid_ids, num_tokens, model_dim, inter_dim,
                    size_expert_ids, experts, topk, tile_m, doweight, out_dtype, 0, a_layout, a_scale_layout,
                    FLYMOE_IMPL_TCGEN05, FLYMOE_SCALE_BLOCK128, FLYMOE_E4M3, stream);
}

// ---------------------------------------------------------------------------------------------
// Dense block-scaled GEMM: the stage-2 kernel with one expert, identity routing and plain stores.
namespace flymoe {
__global__ void dense_routing_kernel(int* __restrict__ sorted_ids, int* __restrict__ sorted_expert_ids,
                                     int* __restrict__ num_valid_ids, int m, int rows_padded, int blocks) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < rows_padded) sorted_ids[i] = i < m ? i : ((1 << 24) | m);   // slot 0 of "token" i; pad id beyond M
  if (i < blocks) sorted_expert_ids[i] = 0;
  if (i == 0) { num_valid_ids[0] = rows_padded; num_valid_ids[1] = m; }
}
}  // namespace flymoe

extern "C" int64_t flymoe_blockscale_gemm_workspace_elems(int m, int tile_m) {
  if (m <= 0 || tile_m <= 0) return 0;
  const int64_t blocks = (int64_t(m) + tile_m - 1) / tile_m;
  return blocks * tile_m + blocks + 2;
}

extern "C" int flymoe_blockscale_gemm(void* c, const void* a, const float* scale_a, int64_t sa_stride,
                                      const void* b, const float* scale_b, int32_t* workspace,
                                      int64_t workspace_elems, int m, int n, int k, int tile_m, int out_dtype,
                                      void* stream) {
  using namespace flymoe;
  FLYMOE_REQUIRE(m >= 0 && m < (1 << 24), "blockscale_gemm: M out of range");
  FLYMOE_REQUIRE(n > 0 && n % 64 == 0, "blockscale_gemm: N must be a positive multiple of 64");
  FLYMOE_REQUIRE(k > 0 && k % 128 == 0, "blockscale_gemm: K must be a positive multiple of 128");
  FLYMOE_REQUIRE(tile_m == 16 || tile_m == 32 || tile_m == 64 || tile_m == 128,
                 "blockscale_gemm: tile_m must be 16, 32, 64 or 128");
  FLYMOE_REQUIRE(out_dtype == FLYMOE_F16 || out_dtype == FLYMOE_BF16, "blockscale_gemm: out_dtype must be F16 or BF16");
  if (m == 0) return FLYMOE_OK;
  FLYMOE_REQUIRE(c && a && scale_a && b && scale_b && workspace, "blockscale_gemm: null pointer");
  FLYMOE_REQUIRE(aligned16(c) && aligned16(a) && aligned16(b), "blockscale_gemm: c/a/b must be 16-byte aligned");
  FLYMOE_REQUIRE(sa_stride >= m, "blockscale_gemm: sa_stride smaller than M");
  FLYMOE_REQUIRE(workspace_elems >= flymoe_blockscale_gemm_workspace_elems(m, tile_m),
                 "blockscale_gemm: workspace too small");
  int* status = device_status_ptr();
  FLYMOE_REQUIRE(status != nullptr, "blockscale_gemm: no CUDA device");
  const int blocks = (m + tile_m - 1) / tile_m;
  const int rows_padded = blocks * tile_m;
  int* sorted_ids = workspace;
  int* sorted_expert_ids = workspace + rows_padded;
  int* num_valid_ids = sorted_expert_ids + blocks;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  dense_routing_kernel<<<(rows_padded + 255) / 256, 256, 0, s>>>(sorted_ids, sorted_expert_ids, num_valid_ids, m,
                                                                 rows_padded, blocks);
  FLYMOE_CUDA_CHECK(cudaGetLastError());

  GemmArgs g;
  g.a = static_cast<const uint8_t*>(a);
  g.scale_a = scale_a;
  g.sa_stride = sa_stride;
  g.sa_row_stride = 1;
  g.a_layout = FLYMOE_ROWS_SORTED;
  g.a_scale_layout = FLYMOE_ROWS_SORTED;
  g.a_rows = m;                       // rows beyond M are filled with zeros by the TMA unit, never read from memory
  g.w = static_cast<const uint8_t*>(b);
  g.scale_w = scale_b;
  g.sorted_ids = sorted_ids;
  g.sorted_expert_ids = sorted_expert_ids;
  g.sorted_weights = nullptr;
  g.num_valid_ids = num_valid_ids;
  g.out = c;
  g.out_scale = nullptr;
  g.out_scale_stride = 0;
  g.out_dtype = out_dtype;
  g.out_layout = FLYMOE_ROWS_BY_PAIR;
  g.accumulate = 0;
  g.row_dst = nullptr;
  g.doweight = 0;
  g.scaling = FLYMOE_SCALE_BLOCK128;
  g.in_dtype = FLYMOE_E4M3;
  g.num_tokens = m;
  g.topk = 1;
  g.experts = 1;
  g.n_dim = n;
  g.k_dim = k;
  g.size_expert_ids = blocks;
  g.tile_m = tile_m;
  g.status = status;
  return launch_gemm_sm100(2, g, s);
}
