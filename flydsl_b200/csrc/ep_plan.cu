// Expert-parallel step planning on the device: rows per expert from the sorted list, and -- from the
// all-gathered rows-per-(rank, expert) matrix -- everything one rank needs for a step whose dispatch and
// combine are peer stores: where each of its own rows lands in the owners' operand buffers, and the
// layout of the rows it receives (sorted ids, block experts, extent, return address of every row).
// The same arithmetic as the host-side planner of the Python layer, so a step needs no host round trip.
#include <algorithm>

#include "common.cuh"

namespace flymoe {

constexpr int kPlanMaxWorld = 8;
constexpr int kPlanMaxExperts = 1024;

// counts[e] = number of rows of the ascending per-row expert list that equal e (two binary searches).
__global__ void __launch_bounds__(256)
expert_counts_kernel(const int* __restrict__ row_expert, const int* __restrict__ num_valid_ids,
                     long long* __restrict__ counts, int experts, int max_rows) {
  const int e = blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= experts) return;
  const int n = min(__ldg(num_valid_ids), max_rows);
  int lo = 0, hi = n;                       // first row with expert >= e
  while (lo < hi) { const int mid = (lo + hi) >> 1; if (__ldg(row_expert + mid) < e) lo = mid + 1; else hi = mid; }
  const int first = lo;
  hi = n;                                   // first row with expert > e
  while (lo < hi) { const int mid = (lo + hi) >> 1; if (__ldg(row_expert + mid) <= e) lo = mid + 1; else hi = mid; }
  counts[e] = lo - first;
}

struct PlanArgs {
  const long long* counts;      // [world, experts]
  const long long* peer_base;   // [world] byte address of every rank's peer-visible buffer
  long long off_x, off_scale, off_back;
  long long* dst_x;             // [experts]
  long long* dst_scale;         // [experts]
  long long* pos_base;          // [experts]
  int* seg;                     // workspace: [per_rank + 1] layout start of each local expert, then
                                // [per_rank * world] rows from each source, then [per_rank * world] first source row
  int* num_valid_ids;           // [2]
  int world, rank, experts, per_rank, unit, model_dim;
  long long cap_rows;
};

// One block.  Thread e owns expert e for the per-expert quantities; the per-source and per-owner prefix
// sums are short serial loops of one thread each (world <= 8 of them).
__global__ void __launch_bounds__(1024)
ep_plan_tables_kernel(PlanArgs p) {
  __shared__ int own_start[kPlanMaxWorld][kPlanMaxExperts];   // start of expert e in source s's sorted order
  __shared__ int start[kPlanMaxExperts];                      // start of expert e in its owner's padded layout
  __shared__ int padded[kPlanMaxExperts];
  __shared__ int extent[kPlanMaxWorld];
  const int tid = threadIdx.x;
  const int W = p.world, E = p.experts, per = p.per_rank;
  for (int e = tid; e < E; e += blockDim.x) {
    long long tot = 0;
    for (int s = 0; s < W; ++s) tot += p.counts[(long long)s * E + e];
    padded[e] = int((tot + p.unit - 1) / p.unit * p.unit);
  }
  if (tid < W) {
    int run = 0;
    for (int e = 0; e < E; ++e) { own_start[tid][e] = run; run += int(p.counts[(long long)tid * E + e]); }
  }
  __syncthreads();
  if (tid < W) {
    int run = 0;
    for (int e = tid * per; e < (tid + 1) * per; ++e) { start[e] = run; run += padded[e]; }
    extent[tid] = run;
  }
  __syncthreads();
  for (int e = tid; e < E; e += blockDim.x) {
    long long before = 0;                   // rows of expert e from sources in front of this rank
    for (int s = 0; s < p.rank; ++s) before += p.counts[(long long)s * E + e];
    const long long pb = (long long)start[e] + before - own_start[p.rank][e];
    const long long base = p.peer_base[e / per];
    p.pos_base[e] = pb;
    p.dst_x[e] = base + p.off_x + pb * p.model_dim;
    p.dst_scale[e] = base + p.off_scale + pb * (p.model_dim / 128) * 4;
  }
  const int lo = p.rank * per;
  int* seg_start = p.seg;
  int* seg_count = p.seg + per + 1;
  int* seg_row = seg_count + per * W;
  for (int le = tid; le < per; le += blockDim.x) {
    seg_start[le] = start[lo + le];
    for (int s = 0; s < W; ++s) {
      seg_count[le * W + s] = int(p.counts[(long long)s * E + lo + le]);
      seg_row[le * W + s] = own_start[s][lo + le];
    }
  }
  if (tid == 0) {
    seg_start[per] = extent[p.rank];
    const int rows = int(min((long long)extent[p.rank], p.cap_rows));
    p.num_valid_ids[0] = rows;
    p.num_valid_ids[1] = rows;
  }
}

// One thread per row of this rank's operand buffer (cap_rows of them).
__global__ void __launch_bounds__(256)
ep_plan_rows_kernel(const int* __restrict__ seg, const long long* __restrict__ peer_base, long long off_back,
                    int* __restrict__ sorted_ids, int* __restrict__ sorted_expert_ids,
                    long long* __restrict__ row_dst, int world, int per_rank, int unit, int model_dim,
                    long long cap_rows) {
  const int* seg_start = seg;
  const int* seg_count = seg + per_rank + 1;
  const int* seg_row = seg_count + per_rank * world;
  const int extent = min((long long)__ldg(seg_start + per_rank), cap_rows);
  const int pad_id = (1 << 24) | int(cap_rows);
  for (long long pos = (long long)blockIdx.x * blockDim.x + threadIdx.x; pos < cap_rows;
       pos += (long long)gridDim.x * blockDim.x) {
    // local expert whose padded range holds pos (clamped to the last one beyond the layout)
    int lo = 0, hi = per_rank;              // largest le with seg_start[le] <= pos
    while (hi - lo > 1) { const int mid = (lo + hi) >> 1; if (__ldg(seg_start + mid) <= pos) lo = mid; else hi = mid; }
    const int le = lo;
    int id = pad_id;
    long long dst = 0;
    if (pos < extent) {
      int off = int(pos) - __ldg(seg_start + le);
      for (int s = 0; s < world; ++s) {
        const int c = __ldg(seg_count + le * world + s);
        if (off < c) {
          id = int(pos);
          dst = __ldg(peer_base + s) + off_back + (long long)(__ldg(seg_row + le * world + s) + off) * model_dim * 2;
          break;
        }
        off -= c;
      }
    }
    sorted_ids[pos] = id;
    row_dst[pos] = dst;
    if (pos % unit == 0) sorted_expert_ids[pos / unit] = le;
  }
}

}  // namespace flymoe

extern "C" int flymoe_expert_counts(const int32_t* row_expert, const int32_t* num_valid_ids, int64_t* counts,
                                    int experts, int max_rows, void* stream) {
  using namespace flymoe;
  FLYMOE_REQUIRE(experts >= 1 && max_rows >= 0, "expert_counts: bad sizes");
  FLYMOE_REQUIRE(row_expert && num_valid_ids && counts, "expert_counts: null pointer");
  expert_counts_kernel<<<ceil_div(experts, 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      row_expert, num_valid_ids, reinterpret_cast<long long*>(counts), experts, max_rows);
  FLYMOE_CUDA_CHECK(cudaGetLastError());
  return FLYMOE_OK;
}

extern "C" int64_t flymoe_ep_plan_workspace_elems(int world, int experts) {
  if (world < 1 || experts < world || experts % world != 0) return 0;
  const int64_t per = experts / world;
  return per + 1 + 2 * per * world;
}

extern "C" int flymoe_ep_plan_direct(const int64_t* counts, const int64_t* peer_base, int64_t off_x,
                                     int64_t off_scale, int64_t off_back, int64_t* dst_x, int64_t* dst_scale,
                                     int64_t* pos_base, int32_t* sorted_ids, int32_t* sorted_expert_ids,
                                     int32_t* num_valid_ids, int64_t* row_dst, int32_t* workspace,
                                     int64_t workspace_elems, int world, int rank, int experts, int unit,
                                     int model_dim, int64_t cap_rows, void* stream) {
  using namespace flymoe;
  FLYMOE_REQUIRE(world >= 1 && world <= kPlanMaxWorld, "ep_plan_direct: world must be in [1, 8]");
  FLYMOE_REQUIRE(experts >= world && experts <= kPlanMaxExperts && experts % world == 0,
                 "ep_plan_direct: experts must be a multiple of world, at most 1024");
  FLYMOE_REQUIRE(rank >= 0 && rank < world, "ep_plan_direct: rank out of range");
  FLYMOE_REQUIRE(unit >= 1 && cap_rows >= 0 && cap_rows % unit == 0 && cap_rows < (1 << 24),
                 "ep_plan_direct: cap_rows must be a multiple of unit below 2^24");
  FLYMOE_REQUIRE(model_dim > 0 && model_dim % 128 == 0, "ep_plan_direct: model_dim must be a positive multiple of 128");
  FLYMOE_REQUIRE(counts && peer_base && dst_x && dst_scale && pos_base && sorted_ids && sorted_expert_ids &&
                     num_valid_ids && row_dst && workspace, "ep_plan_direct: null pointer");
  FLYMOE_REQUIRE(workspace_elems >= flymoe_ep_plan_workspace_elems(world, experts), "ep_plan_direct: workspace too small");
  PlanArgs p;
  p.counts = reinterpret_cast<const long long*>(counts);
  p.peer_base = reinterpret_cast<const long long*>(peer_base);
  p.off_x = off_x; p.off_scale = off_scale; p.off_back = off_back;
  p.dst_x = reinterpret_cast<long long*>(dst_x);
  p.dst_scale = reinterpret_cast<long long*>(dst_scale);
  p.pos_base = reinterpret_cast<long long*>(pos_base);
  p.seg = workspace;
  p.num_valid_ids = num_valid_ids;
  p.world = world; p.rank = rank; p.experts = experts; p.per_rank = experts / world; p.unit = unit;
  p.model_dim = model_dim; p.cap_rows = cap_rows;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  ep_plan_tables_kernel<<<1, 1024, 0, s>>>(p);
  FLYMOE_CUDA_CHECK(cudaGetLastError());
  if (cap_rows > 0) {
    const int blocks = int(std::min<long long>((cap_rows + 255) / 256, (long long)sm_count() * 4));
    ep_plan_rows_kernel<<<blocks, 256, 0, s>>>(workspace, p.peer_base, off_back, sorted_ids, sorted_expert_ids,
                                                reinterpret_cast<long long*>(row_dst), world, p.per_rank, unit, model_dim,
                                                cap_rows);
    FLYMOE_CUDA_CHECK(cudaGetLastError());
  }
  return FLYMOE_OK;
}
