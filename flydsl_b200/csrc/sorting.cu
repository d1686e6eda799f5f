// Token-to-expert counting sort with per-expert padding (stable: experts ascending,
// tokens ascending within an expert).
//
// The (token, slot) pairs are cut into contiguous segments, one per warp.  Each warp
// builds a shared-memory histogram of its segment; an exclusive prefix over segments
// gives every warp its write cursor per expert, and a warp-level match gives each
// pair its rank inside a 32-pair step, so the scatter is deterministic.
//   * P <= kOneBlockMaxPairs : one launch, one block, everything in shared memory.
//   * otherwise              : count (grid) -> scan (one block) -> scatter (grid),
//                              per-segment histograms kept in caller-provided scratch.
#include <stdio.h>

#include "common.cuh"

namespace flymoe {

constexpr int kSortThreads = 256;
constexpr int kSortWarps = kSortThreads / 32;
constexpr int kOneBlockMaxPairs = 8192;
constexpr int kSegPairs = 128;       // pairs per warp segment on the multi-block path
constexpr int kMaxExperts = 1024;

struct SortArgs {
  const int* topk_ids;
  const float* topk_weights;
  int* sorted_ids;
  float* sorted_weights;
  int* sorted_expert_ids;
  int* num_valid_ids;
  const int* expert_mask;
  int* ws_counts;   // [nseg][E] on the multi-block path
  int* ws_base;     // [E]
  int num_tokens, num_experts, topk, unit_size;
  int num_pairs, seg_len, nseg;
  int sorted_capacity, expert_ids_capacity;
};

__device__ __forceinline__ bool pair_expert(const SortArgs& a, int p, int p_end, int& e) {
  if (p >= p_end) return false;
  e = __ldg(a.topk_ids + p);
  if (e < 0 || e >= a.num_experts) return false;
  if (a.expert_mask != nullptr && __ldg(a.expert_mask + e) == 0) return false;
  return true;
}

// Histogram of one warp's segment into cnt[E] (shared memory, zeroed by the caller).
__device__ __forceinline__ void warp_count(const SortArgs& a, int seg, int* cnt, int lane) {
  const int p0 = seg * a.seg_len;
  const int p1 = min(p0 + a.seg_len, a.num_pairs);
  for (int p = p0 + lane; p < p1; p += 32) {
    int e;
    if (pair_expert(a, p, p1, e)) atomicAdd(cnt + e, 1);
  }
}

// Scatter of one warp's segment; cur[E] holds this warp's next write offset per expert
// (relative to the expert's base), base[E] the first sorted row of each expert.
__device__ __forceinline__ void warp_scatter(const SortArgs& a, int seg, int* cur, const int* base,
                                             int lane) {
  const int p0 = seg * a.seg_len;
  const int p1 = min(p0 + a.seg_len, a.num_pairs);
  const unsigned lt_mask = (1u << lane) - 1u;
  for (int pb = p0; pb < p1; pb += 32) {
    const int p = pb + lane;
    int e = 0;
    const bool ok = pair_expert(a, p, p1, e);
    const int key = ok ? e : (kMaxExperts + lane);
    const unsigned grp = __match_any_sync(0xffffffffu, key);
    int c = 0;
    if (ok) c = cur[e];
    __syncwarp();
    if (ok && (grp & lt_mask) == 0) cur[e] = c + __popc(grp);
    __syncwarp();
    if (ok) {
      const int pos = base[e] + c + __popc(grp & lt_mask);
      const int token = p / a.topk;
      const int slot = p - token * a.topk;
      a.sorted_ids[pos] = (slot << 24) | token;
      a.sorted_weights[pos] = __ldg(a.topk_weights + p);
    }
  }
}

// Block-wide: totals per expert -> padded bases, block->expert table, valid row count.
// tot[E] in shared memory holds the pair count per expert on entry; on exit base[E]
// holds each expert's first sorted row.  Pad rows inside the valid range receive the
// sentinel id and weight 0; rows at or beyond the valid count are left untouched.
// scratch: 2 * 32 ints of shared memory.
__device__ void block_layout(const SortArgs& a, const int* tot, int* base, int* scratch) {
  const int tid = threadIdx.x, nthr = blockDim.x;
  const int E = a.num_experts, U = a.unit_size;
  const int ept = (E + nthr - 1) / nthr;          // experts per thread (contiguous)
  const int e0 = min(tid * ept, E), e1 = min(e0 + ept, E);
  int rows = 0, disabled = 0;
  for (int e = e0; e < e1; ++e) {
    rows += ((tot[e] + U - 1) / U) * U;
    disabled += (a.expert_mask != nullptr && __ldg(a.expert_mask + e) == 0) ? 1 : 0;
  }
  // exclusive block scan of (rows, disabled) over threads
  const int lane = tid & 31, warp = tid >> 5, nwarp = (nthr + 31) >> 5;
  int r_inc = rows, d_inc = disabled;
#pragma unroll
  for (int off = 1; off < 32; off <<= 1) {
    const int r2 = __shfl_up_sync(0xffffffffu, r_inc, off);
    const int d2 = __shfl_up_sync(0xffffffffu, d_inc, off);
    if (lane >= off) { r_inc += r2; d_inc += d2; }
  }
  if (lane == 31) { scratch[warp] = r_inc; scratch[32 + warp] = d_inc; }
  __syncthreads();
  if (warp == 0) {
    int r = lane < nwarp ? scratch[lane] : 0, d = lane < nwarp ? scratch[32 + lane] : 0;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
      const int r2 = __shfl_up_sync(0xffffffffu, r, off);
      const int d2 = __shfl_up_sync(0xffffffffu, d, off);
      if (lane >= off) { r += r2; d += d2; }
    }
    scratch[lane] = r; scratch[32 + lane] = d;   // inclusive over warps
  }
  __syncthreads();
  int row = r_inc - rows + (warp > 0 ? scratch[warp - 1] : 0);
  int dis = d_inc - disabled + (warp > 0 ? scratch[32 + warp - 1] : 0);
  const int total_rows = scratch[nwarp - 1];
  const int sentinel = (a.topk << 24) | a.num_tokens;   // used by the pad fill below
  for (int e = e0; e < e1; ++e) {
    const bool off = (a.expert_mask != nullptr && __ldg(a.expert_mask + e) == 0);
    base[e] = row;
    const int nb = (tot[e] + U - 1) / U;
    const int b0 = row / U;
    for (int b = 0; b < nb; ++b)
      if (b0 + b < a.expert_ids_capacity) a.sorted_expert_ids[b0 + b] = e - dis;
    row += nb * U;
    dis += off ? 1 : 0;
  }
  for (int b = total_rows / U + tid; b < a.expert_ids_capacity; b += nthr) a.sorted_expert_ids[b] = -1;
  if (tid == 0) { a.num_valid_ids[0] = total_rows; a.num_valid_ids[1] = a.num_tokens; }
  __syncthreads();
  // pad rows (sentinel id, weight 0) of every expert: one warp per expert, lanes across the pad range
  for (int e = warp; e < E; e += nwarp) {
    const int first = base[e] + tot[e];
    const int last = base[e] + ((tot[e] + U - 1) / U) * U;
    for (int i = first + lane; i < last; i += 32) {
      a.sorted_ids[i] = sentinel;
      a.sorted_weights[i] = 0.f;
    }
  }
}

__global__ void __launch_bounds__(kSortThreads) moe_sort_oneblock_kernel(SortArgs a) {
  extern __shared__ int smem[];
  const int E = a.num_experts;
  int* cnt = smem;                       // [kSortWarps][E]
  int* tot = cnt + kSortWarps * E;       // [E]
  int* base = tot + E;                   // [E]
  int* scratch = base + E;               // [64]
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;

  for (int i = tid; i < kSortWarps * E; i += kSortThreads) cnt[i] = 0;
  __syncthreads();
  warp_count(a, warp, cnt + warp * E, lane);
  __syncthreads();
  for (int e = tid; e < E; e += kSortThreads) {
    int run = 0;
#pragma unroll
    for (int w = 0; w < kSortWarps; ++w) {
      const int c = cnt[w * E + e];
      cnt[w * E + e] = run;
      run += c;
    }
    tot[e] = run;
  }
  __syncthreads();
  block_layout(a, tot, base, scratch);
  warp_scatter(a, warp, cnt + warp * E, base, lane);
}

// Multi-block path, step 1: per-segment histograms to scratch.
__global__ void __launch_bounds__(kSortThreads) moe_sort_count_kernel(SortArgs a) {
  extern __shared__ int smem[];
  const int E = a.num_experts;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  int* cnt = smem + warp * E;
  for (int i = tid; i < kSortWarps * E; i += kSortThreads) smem[i] = 0;
  __syncthreads();
  const int seg = blockIdx.x * kSortWarps + warp;
  if (seg < a.nseg) {
    warp_count(a, seg, cnt, lane);
    __syncwarp();
    for (int e = lane; e < E; e += 32) a.ws_counts[size_t(seg) * E + e] = cnt[e];
  }
}

// Step 2 (one block of 1024 threads): exclusive prefix over segments per expert, then the expert
// layout.  The segment axis is cut into `parts` contiguous ranges handled by different threads of
// the same expert (parts * E <= 1024), so the serial walk per thread is nseg / parts long.
__global__ void __launch_bounds__(1024) moe_sort_scan_kernel(SortArgs a) {
  __shared__ int tot[kMaxExperts];
  __shared__ int base[kMaxExperts];
  __shared__ int scratch[64];
  __shared__ int part_sum[1024];
  const int E = a.num_experts;
  int parts = 1;
  while (parts * 2 * E <= 1024 && parts * 2 <= a.nseg) parts *= 2;
  const int per_part = (a.nseg + parts - 1) / parts;
  const int e = threadIdx.x % E, part = threadIdx.x / E;
  const bool active = part < parts && threadIdx.x < parts * E;
  const int s0 = min(part * per_part, a.nseg), s1 = min(s0 + per_part, a.nseg);
  int sum = 0;
  if (active) {
#pragma unroll 8
    for (int s = s0; s < s1; ++s) sum += a.ws_counts[size_t(s) * E + e];
    part_sum[part * E + e] = sum;
  }
  __syncthreads();
  if (active) {
    int run = 0;
    for (int q = 0; q < part; ++q) run += part_sum[q * E + e];
    if (part == parts - 1) tot[e] = run + sum;
#pragma unroll 4
    for (int s = s0; s < s1; ++s) {
      const int c = a.ws_counts[size_t(s) * E + e];
      a.ws_counts[size_t(s) * E + e] = run;
      run += c;
    }
  }
  __syncthreads();
  block_layout(a, tot, base, scratch);
  for (int x = threadIdx.x; x < E; x += blockDim.x) a.ws_base[x] = base[x];
}

// Step 3: scatter.
__global__ void __launch_bounds__(kSortThreads) moe_sort_scatter_kernel(SortArgs a) {
  extern __shared__ int smem[];
  const int E = a.num_experts;
  int* base = smem;                      // [E]
  int* cur_all = smem + E;               // [kSortWarps][E]
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  for (int e = tid; e < E; e += kSortThreads) base[e] = a.ws_base[e];
  const int seg = blockIdx.x * kSortWarps + warp;
  int* cur = cur_all + warp * E;
  if (seg < a.nseg)
    for (int e = lane; e < E; e += 32) cur[e] = a.ws_counts[size_t(seg) * E + e];
  __syncthreads();
  if (seg < a.nseg) warp_scatter(a, seg, cur, base, lane);
}

static void sort_plan(int num_pairs, int* seg_len, int* nseg, bool* one_block) {
  if (num_pairs <= kOneBlockMaxPairs) {
    *one_block = true;
    int per_warp = ceil_div(num_pairs > 0 ? num_pairs : 1, kSortWarps);
    *seg_len = ceil_div(per_warp, 32) * 32;
    *nseg = kSortWarps;
  } else {
    *one_block = false;
    *seg_len = kSegPairs;
    *nseg = ceil_div(num_pairs, kSegPairs);
  }
}

}  // namespace flymoe

extern "C" int64_t flymoe_moe_sorting_workspace_elems(int num_tokens, int num_experts, int topk,
                                                      int unit_size) {
  (void)unit_size;
  if (num_tokens < 0 || num_experts < 1 || topk < 1) return 0;
  const int64_t pairs = int64_t(num_tokens) * topk;
  if (pairs >= (int64_t(1) << 30))           // beyond what flymoe_moe_sorting accepts: size from the segment length
    return ((pairs + flymoe::kSegPairs - 1) / flymoe::kSegPairs) * num_experts + num_experts;
  int seg_len, nseg;
  bool one_block;
  flymoe::sort_plan(int(pairs), &seg_len, &nseg, &one_block);
  if (one_block) return 0;
  return int64_t(nseg) * num_experts + num_experts;
}

extern "C" int flymoe_moe_sorting(const int32_t* topk_ids, const float* topk_weights,
                                  int32_t* sorted_ids, float* sorted_weights,
                                  int32_t* sorted_expert_ids, int32_t* num_valid_ids, void* moe_buf,
                                  int64_t moe_buf_bytes, const int32_t* expert_mask,
                                  int32_t* workspace, int64_t workspace_elems, int num_tokens,
                                  int num_experts, int topk, int unit_size, void* stream) {
  using namespace flymoe;
  FLYMOE_REQUIRE(num_tokens >= 0 && num_tokens < (1 << 24), "sorting: num_tokens must be in [0, 2^24)");
  FLYMOE_REQUIRE(num_experts >= 1 && num_experts <= kMaxExperts, "sorting: num_experts must be in [1, 1024]");
  FLYMOE_REQUIRE(topk >= 1 && topk <= 255, "sorting: topk must be in [1, 255]");
  // the padded rows total at most pairs + E*(unit-1), which fits the caller's pairs + E*unit - topk
  // buffer only when topk <= E (a token routes to distinct experts)
  FLYMOE_REQUIRE(topk <= num_experts, "sorting: topk must not exceed num_experts");
  FLYMOE_REQUIRE(unit_size >= 1, "sorting: unit_size must be >= 1");
  FLYMOE_REQUIRE(int64_t(num_tokens) * topk < (int64_t(1) << 30), "sorting: too many (token, slot) pairs");
  FLYMOE_REQUIRE(sorted_ids && sorted_weights && sorted_expert_ids && num_valid_ids, "sorting: null output");
  FLYMOE_REQUIRE(num_tokens == 0 || (topk_ids && topk_weights), "sorting: null input");
  cudaStream_t s = static_cast<cudaStream_t>(stream);

  SortArgs a;
  a.topk_ids = topk_ids; a.topk_weights = topk_weights;
  a.sorted_ids = sorted_ids; a.sorted_weights = sorted_weights;
  a.sorted_expert_ids = sorted_expert_ids; a.num_valid_ids = num_valid_ids;
  a.expert_mask = expert_mask;
  a.num_tokens = num_tokens; a.num_experts = num_experts; a.topk = topk; a.unit_size = unit_size;
  a.num_pairs = num_tokens * topk;
  a.sorted_capacity = a.num_pairs + num_experts * unit_size - topk;
  if (a.sorted_capacity < 0) a.sorted_capacity = 0;
  a.expert_ids_capacity = ceil_div(a.sorted_capacity, unit_size);
  bool one_block;
  sort_plan(a.num_pairs, &a.seg_len, &a.nseg, &one_block);
  a.ws_counts = nullptr; a.ws_base = nullptr;

  if (moe_buf != nullptr && moe_buf_bytes > 0)
    FLYMOE_CUDA_CHECK(cudaMemsetAsync(moe_buf, 0, size_t(moe_buf_bytes), s));

  if (one_block) {
    const size_t smem = size_t(kSortWarps + 2) * num_experts * sizeof(int) + 64 * sizeof(int);
    if (smem > 48 * 1024)
      FLYMOE_CUDA_CHECK(cudaFuncSetAttribute(moe_sort_oneblock_kernel,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)));
    moe_sort_oneblock_kernel<<<1, kSortThreads, smem, s>>>(a);
    FLYMOE_CUDA_CHECK(cudaGetLastError());
    return FLYMOE_OK;
  }

  const int64_t need = int64_t(a.nseg) * num_experts + num_experts;
  if (workspace == nullptr || workspace_elems < need) {
    set_last_error_msg("sorting: workspace smaller than flymoe_moe_sorting_workspace_elems()");
    return FLYMOE_ERR_WORKSPACE;
  }
  a.ws_counts = workspace;
  a.ws_base = workspace + int64_t(a.nseg) * num_experts;
  const int nblk = ceil_div(a.nseg, kSortWarps);
  const size_t smem_cnt = size_t(kSortWarps) * num_experts * sizeof(int);
  const size_t smem_sct = size_t(kSortWarps + 1) * num_experts * sizeof(int);
  if (smem_sct > 48 * 1024)
    FLYMOE_CUDA_CHECK(cudaFuncSetAttribute(moe_sort_scatter_kernel,
                                           cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem_sct)));
  moe_sort_count_kernel<<<nblk, kSortThreads, smem_cnt, s>>>(a);
  FLYMOE_CUDA_CHECK(cudaGetLastError());
  moe_sort_scan_kernel<<<1, 1024, 0, s>>>(a);
  FLYMOE_CUDA_CHECK(cudaGetLastError());
  moe_sort_scatter_kernel<<<nblk, kSortThreads, smem_sct, s>>>(a);
  FLYMOE_CUDA_CHECK(cudaGetLastError());
  return FLYMOE_OK;
}

// ---------------------------------------------------------------------------------------
// Allocation-free variant of the sort.
//
// Some hosts of this library may not allocate device memory on their call path at all: a
// serving loop that has handed the whole device heap to its own pool, a plugin running
// inside another framework's memory budget, or code that must not touch the allocator
// because allocation can synchronise the device.  For them the multi-block path's scratch
// lives in the array below, which every GPU that loads the library holds until exit
// (kNoAllocScratchElems * 4 bytes = 4 MiB).
constexpr long long kNoAllocScratchElems = 1ll << 20;
static __device__ __align__(256) int32_t g_sort_scratch[kNoAllocScratchElems];

namespace flymoe {

// In host code `g_sort_scratch` is only a handle for the symbol, not a device address, so
// the address is looked up once per device (with that device current) and cached.
static int noalloc_scratch(int32_t** out) {
  static int32_t* cached[64] = {nullptr};
  int dev = 0;
  FLYMOE_CUDA_CHECK(cudaGetDevice(&dev));
  FLYMOE_REQUIRE(dev >= 0 && dev < 64, "sorting (no-alloc): device ordinal out of range");
  if (cached[dev] == nullptr) {
    int32_t* p = nullptr;
    FLYMOE_CUDA_CHECK(cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_sort_scratch));
    FLYMOE_REQUIRE(p != nullptr, "sorting (no-alloc): scratch symbol has no device address");
    cached[dev] = p;
  }
  *out = cached[dev];
  return FLYMOE_OK;
}

}  // namespace flymoe

extern "C" int64_t flymoe_moe_sorting_noalloc_max_elems(void) { return kNoAllocScratchElems; }

extern "C" int flymoe_moe_sorting_noalloc(const int32_t* topk_ids, const float* topk_weights,
                                          int32_t* sorted_ids, float* sorted_weights,
                                          int32_t* sorted_expert_ids, int32_t* num_valid_ids,
                                          void* moe_buf, int64_t moe_buf_bytes,
                                          const int32_t* expert_mask, int num_tokens, int num_experts,
                                          int topk, int unit_size, void* stream) {
  using namespace flymoe;
  const int64_t need = flymoe_moe_sorting_workspace_elems(num_tokens, num_experts, topk, unit_size);
  if (need > kNoAllocScratchElems) {
    char msg[200];
    snprintf(msg, sizeof(msg),
             "sorting (no-alloc): this problem needs %lld int32 of scratch, the built-in array holds %lld; "
             "use flymoe_moe_sorting with a caller-provided workspace",
             (long long)need, (long long)kNoAllocScratchElems);
    set_last_error_msg(msg);
    return FLYMOE_ERR_WORKSPACE;
  }
  int32_t* scratch = nullptr;
  const int rc = noalloc_scratch(&scratch);
  if (rc != FLYMOE_OK) return rc;
  return flymoe_moe_sorting(topk_ids, topk_weights, sorted_ids, sorted_weights, sorted_expert_ids,
                            num_valid_ids, moe_buf, moe_buf_bytes, expert_mask, scratch,
                            kNoAllocScratchElems, num_tokens, num_experts, topk, unit_size, stream);
}
