// Grouped FP8 (e4m3) GEMM for both MoE stages on sm_100a.
//
// One persistent CTA per SM walks a static sequence of (sorted row block, N tile)
// tiles.  Warp roles (384 threads):
//   warp 0      TMA producer: per 128-wide K block one A box (tile_m sorted rows x 128 B)
//               and 256 weight rows x 128 B into a 4-deep (stage 2: 3-deep) shared-memory
//               ring (128-byte swizzle, K-major).
//   warp 1      MMA issuer: four tcgen05.mma (M=128, N=256, K=32) per K block into one of
//               two 256-column TMEM accumulator stages; tcgen05.commit releases the smem
//               stage and publishes the TMEM stage.
//   warp 2      store warp: sends the finished rows that the epilogue threads parked in
//               shared-memory slots to global memory as bulk stores / bulk reductions
//               (one per slot), so their issue cost is off the epilogue's path.
//   warp 3      row gather (only when the activations are not in sorted-row order): copies the
//               tile's A rows, picked through the sorted-id list, into the ring with cp.async
//               (16 bytes per request, the 128-byte swizzle applied by hand), two K blocks in
//               flight; the TMA producer then fetches the weights only.  Meant for row blocks
//               of 16 or 32 rows; larger ones are gathered ahead of the launch.
//   warps 4-11  epilogue, two warpgroups.  Each thread owns one sorted row (its TMEM lane)
//               and 128 of the tile's 256 accumulator columns.
//
// Two scaling modes (template parameter SCALING):
//   kScaleBlock128   activation scales per (row, 128 K), weight scales per 128x128 block.
//               The scales are arbitrary fp32, so they cannot ride inside the MMA: every
//               K block starts its TMEM stage from zero, and the epilogue folds the K
//               block's partial sums into register accumulators with the product of the
//               row's activation scale and the weight block's scale (packed fma.rn.f32x2).
//   kScalePerToken   one scale per activation row and one per weight row (output
//               column): the MMA accumulates over the whole K range in TMEM and the
//               epilogue drains each tile once.  fp8 e4m3 or int8 operands.
//
// Stage 1 tile: 128 gate rows + 128 up rows of W1 (one quantisation group of the
// output); each warpgroup takes 64 gate + 64 up columns, computes silu(gate)*up and
// either stores f16/bf16 or requantises to e4m3 with the per-row 1x128 scale (row amax
// exchanged between the two warpgroups through shared memory).
// Stage 2 tile: 256 rows of W2; each warpgroup takes 128 columns; every thread multiplies
// its row by the routing weight, parks the 256 bytes in a private shared-memory slot and
// the store warp adds them into out[token] with one bulk reduce (cp.reduce.async.bulk),
// bulk-stores per-pair rows for a later top-k reduce, or (ROW_DST instantiation) stores
// each row to a caller-given address, which may be in a peer GPU's memory.  The same
// kernel with one expert and identity routing is the dense block-scaled GEMM.
//
// Every wait is bounded: when one gives up it raises the CTA's abort flag and the
// device status word, every role drains out, TMEM is released and the kernel returns.
#include <cuda.h>
#include <cudaTypedefs.h>
#include <stdio.h>

#include "common.cuh"
#include "gemm_args.cuh"

namespace flymoe {

constexpr int BM = 128;
constexpr int BN = 256;
constexpr int BK = 128;
// Upper bound on the persistent grid (0 = one CTA per SM).  A caller that overlaps the GEMMs with
// communication kernels leaves those kernels some SMs: a persistent CTA that cannot become resident
// at launch would otherwise run its whole tile list after the others have finished.
static int g_cta_limit = 0;

constexpr int kScaleBlock128 = 0;
constexpr int kScalePerToken = 1;

constexpr int kMaxStages = 4;
// Depth of the shared-memory operand ring.  Stage 2 gives one slot up for a staging area from
// which finished output rows leave by bulk reduce/store (measured: a 3-deep ring is as fast as 4).
template <int STAGE> struct RingDepth { static constexpr int value = STAGE == 1 ? 4 : 3; };
// Per-epilogue-thread staging slot for finished output: stage 2 holds 256 B of 16-bit results,
// stage 1 holds 64 e4m3 codes; 16 B of skew keep 16-byte shared-memory stores conflict-free.
template <int STAGE> struct Staging {
  static constexpr int stride = STAGE == 1 ? 80 : 272;
  static constexpr int bytes = 256 * stride;
};
constexpr int kATileBytes = BM * BK;            // 16 KB
constexpr int kBTileBytes = BN * BK;            // 32 KB
constexpr int kStageBytes = kATileBytes + kBTileBytes;
constexpr int kAccStages = 2;
constexpr int kTmemCols = 512;
constexpr int kNumThreads = 384;
constexpr int kEpilogueWarps = 8;
constexpr unsigned long long kWaitLimitNs = 4000000000ull;   // 4 s

struct __align__(16) SmemCtrl {
  unsigned long long full[kMaxStages];
  unsigned long long empty[kMaxStages];
  unsigned long long tmem_full[kAccStages];
  unsigned long long tmem_empty[kAccStages];
  unsigned long long amax_bar[2];
  unsigned long long stg_full;                  // epilogue warps -> store warp: slots and destinations written
  unsigned long long stg_free;                  // store warp -> epilogue warps: slots have been read
  unsigned long long stg_dst[256];              // per epilogue thread: global address of its row segment, 0 = none
  uint32_t tmem_base;
  int abort_flag;
  float amax[2][2][BM];
};
template <int STAGE> constexpr size_t smem_bytes() {
  return size_t(RingDepth<STAGE>::value) * kStageBytes + Staging<STAGE>::bytes + sizeof(SmemCtrl) + 1024;
}
static_assert(smem_bytes<1>() <= 232448 && smem_bytes<2>() <= 232448, "shared memory budget of one SM exceeded");

// Optional whole-kernel wait accounting (build with -DFLYMOE_PROF, `python -m flydsl_b200.build
// --prof`): every CTA's producer thread, MMA thread and first epilogue thread add up the cycles they
// spend in each wait and write the sums once at the end; flymoe_prof_read() copies them out as
// [CTA][role][8] int64 (`python bench.py --wait-accounting` prints the means).
#ifdef FLYMOE_PROF
__device__ long long g_prof[256][3][8];
#define PROF_DECL long long prof_t0 = clock64(), prof_s = 0, prof_w[6] = {0, 0, 0, 0, 0, 0};
#define PROF_START prof_s = clock64();
#define PROF_STOP(i) prof_w[i] += clock64() - prof_s;
#define PROF_COUNT(i) prof_w[i] += 1;
#define PROF_WRITE(role)                                                         \
  do {                                                                           \
    if (blockIdx.x < 256) {                                                      \
      g_prof[blockIdx.x][role][0] = clock64() - prof_t0;                         \
      for (int pi = 0; pi < 6; ++pi) g_prof[blockIdx.x][role][1 + pi] = prof_w[pi]; \
    }                                                                            \
  } while (0)
#else
#define PROF_DECL
#define PROF_START
#define PROF_STOP(i)
#define PROF_COUNT(i)
#define PROF_WRITE(role) do {} while (0)
#endif

// ------------------------------------------------------------------------------ PTX
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
// Arrive without release ordering: for hand-offs that publish no memory (a TMEM stage whose
// loads have already completed), so the arrive need not wait for this thread's loads in flight.
__device__ __forceinline__ void mbar_arrive_relaxed(uint32_t bar) {
  asm volatile("mbarrier.arrive.relaxed.cta.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ uint32_t mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t done;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(done) : "r"(bar), "r"(parity) : "memory");
  return done;
}
__device__ __forceinline__ unsigned long long global_timer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}
// Bounded wait.  Returns false when the CTA is aborting or the time limit ran out.
// `backoff_ns` > 0 makes a role that has slack sleep between polls instead of competing for
// issue slots with the epilogue warps of its scheduler partition.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag,
                                          int* status, int code, unsigned backoff_ns = 0,
                                          unsigned long long limit_ns = kWaitLimitNs) {
  if (mbar_try_wait(bar, parity)) return true;
  const unsigned long long t0 = global_timer_ns();
#pragma unroll 1
  for (uint32_t it = 1;; ++it) {
    if (mbar_try_wait(bar, parity)) return true;
    if (backoff_ns) __nanosleep(backoff_ns);
    if ((it & 0xFF) == 0) {
      if (*abort_flag) return false;
      if (global_timer_ns() - t0 > limit_ns) {
        *abort_flag = 1;
        atomicCAS(status, 0, code);
        return false;
      }
    }
  }
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1) : "memory");
}
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1,
                                            int c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2) : "memory");
}
__device__ __forceinline__ void tcgen05_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tcgen05_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void umma_f8(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                        uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_i8(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                        uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                         uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar)
               : "memory");
}
__device__ __forceinline__ void tmem_ld_x32(uint32_t taddr, uint32_t* v) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
        "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]),
        "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]),
        "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
      : "r"(taddr) : "memory");
}
__device__ __forceinline__ unsigned long long pack_f32x2(float x) {
  unsigned long long r;
  asm("mov.b64 %0, {%1, %1};" : "=l"(r) : "f"(x));
  return r;
}
__device__ __forceinline__ void unpack_f32x2(unsigned long long p, float& lo, float& hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(p));
}
// acc.lo += v0 * c.lo ; acc.hi += v1 * c.hi  (one instruction on sm_100)
__device__ __forceinline__ void ffma2(unsigned long long& acc, uint32_t v0, uint32_t v1, unsigned long long c) {
  unsigned long long v;
  asm("mov.b64 %0, {%1, %2};" : "=l"(v) : "r"(v0), "r"(v1));
  asm("fma.rn.f32x2 %0, %1, %2, %0;" : "+l"(acc) : "l"(v), "l"(c));
}
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float fast_rcp(float x) {
  float y;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// K-major, 128-byte-swizzled operand tile: 8-row groups 1024 B apart.
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= uint64_t((smem_addr >> 4) & 0x3FFF);          // start address
  d |= uint64_t(1) << 16;                            // leading byte offset (unused with swizzle)
  d |= uint64_t((1024 >> 4) & 0x3FFF) << 32;         // stride byte offset
  d |= uint64_t(1) << 46;                            // descriptor version (sm_100)
  d |= uint64_t(2) << 61;                            // SWIZZLE_128B
  return d;
}
// Instruction descriptors, both operands K-major, M=128, N=256:
// kind::f8f6f4 with A=B=e4m3 (format 0) and D=f32 (format 1); kind::i8 with A=B=s8 (format 1) and D=s32 (format 2);
// kind::f16 with A=B=f16 (format 0) or bf16 (format 1) and D=f32.  One instruction covers 32 bytes of K in
// every kind (32 one-byte or 16 two-byte elements), so a 128-byte K block is four instructions in all of them.
constexpr uint32_t kInstrDescShape = (uint32_t(BN >> 3) << 17) | (uint32_t(BM >> 4) << 24);
constexpr uint32_t kInstrDescF8 = (1u << 4) | (0u << 7) | (0u << 10) | kInstrDescShape;
constexpr uint32_t kInstrDescI8 = (2u << 4) | (1u << 7) | (1u << 10) | kInstrDescShape;
constexpr uint32_t kInstrDescF16 = (1u << 4) | (0u << 7) | (0u << 10) | kInstrDescShape;
constexpr uint32_t kInstrDescBF16 = (1u << 4) | (1u << 7) | (1u << 10) | kInstrDescShape;

// Bulk operations from a staging slot to a contiguous global row segment (16-byte aligned, size % 16 == 0).
__device__ __forceinline__ void bulk_reduce_add_bf16(void* g, uint32_t s, uint32_t bytes) {
  asm volatile("cp.reduce.async.bulk.global.shared::cta.bulk_group.add.noftz.bf16 [%0], [%1], %2;"
               ::"l"(g), "r"(s), "r"(bytes) : "memory");
}
__device__ __forceinline__ void bulk_reduce_add_f16(void* g, uint32_t s, uint32_t bytes) {
  asm volatile("cp.reduce.async.bulk.global.shared::cta.bulk_group.add.noftz.f16 [%0], [%1], %2;"
               ::"l"(g), "r"(s), "r"(bytes) : "memory");
}
__device__ __forceinline__ void bulk_store(void* g, uint32_t s, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(g), "r"(s), "r"(bytes) : "memory");
}
__device__ __forceinline__ void bulk_wait_read_all() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void red_add_v4_f32(float* p, float a, float b, float c, float d) {
  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(p), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}
// ------------------------------------------------------------------------------ tiles
struct TileSched {
  int num_mblocks, num_ntiles, total, group_m;
  __device__ __forceinline__ void decode(int t, int& mb, int& n) const {
    const int per_group = group_m * num_ntiles;
    const int bg = t / per_group;
    const int rem = t - bg * per_group;
    const int gs = min(group_m, num_mblocks - bg * group_m);
    n = rem / gs;
    mb = bg * group_m + (rem - n * gs);
  }
};

// ROW_DST (stage 2 only): every output row goes to a caller-given address instead of out[t*k+s].  A
// separate instantiation, so that the common kernel's register allocation is not touched.
// GATHER: a separate instantiation, so that the kernels reading sorted rows keep their register allocation.
template <int STAGE, bool ROW_DST, int SCALING, bool GATHER>
__global__ void __launch_bounds__(kNumThreads, 1)
moe_gemm_sm100_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                      const GemmArgs a, const int group_m) {
  extern __shared__ uint8_t smem_dyn[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~uintptr_t(1023));
  constexpr int kStages = RingDepth<STAGE>::value;
  uint8_t* staging = smem + size_t(kStages) * kStageBytes;
  SmemCtrl* ctrl = reinterpret_cast<SmemCtrl*>(staging + Staging<STAGE>::bytes);
  volatile int* abort_flag = &ctrl->abort_flag;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int KB = a.k_dim / BK;

  const int valid_rows = min(__ldg(a.num_valid_ids), a.size_expert_ids * a.tile_m);
  // A rows are fetched by index (row = token, or token*topk+slot) instead of by one TMA box per K block
  constexpr bool gather = GATHER;
  // Outputs that leave through the staging slots (everything except 16-bit stage-1 and fp32 stage-2 output)
  const bool uses_staging = STAGE == 1 ? a.out_dtype == FLYMOE_E4M3 : a.out_dtype != FLYMOE_F32;
  TileSched sched;
  sched.num_mblocks = (valid_rows + a.tile_m - 1) / a.tile_m;
  sched.num_ntiles = STAGE == 1 ? a.n_dim / 128 : (a.n_dim + BN - 1) / BN;
  sched.total = sched.num_mblocks * sched.num_ntiles;
  sched.group_m = group_m;

  if (threadIdx.x == 0) {
    for (int i = 0; i < kStages; ++i) {
      mbar_init(smem_u32(&ctrl->full[i]), gather ? 2 : 1);     // TMA thread (+ the gather warp)
      mbar_init(smem_u32(&ctrl->empty[i]), 1);
    }
    for (int i = 0; i < kAccStages; ++i) {
      mbar_init(smem_u32(&ctrl->tmem_full[i]), 1);
      mbar_init(smem_u32(&ctrl->tmem_empty[i]), kEpilogueWarps);
    }
    mbar_init(smem_u32(&ctrl->amax_bar[0]), kEpilogueWarps);
    mbar_init(smem_u32(&ctrl->amax_bar[1]), kEpilogueWarps);
    mbar_init(smem_u32(&ctrl->stg_full), kEpilogueWarps);
    mbar_init(smem_u32(&ctrl->stg_free), 1);
    ctrl->abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                 ::"r"(smem_u32(&ctrl->tmem_base)), "r"(uint32_t(kTmemCols)) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem_base = ctrl->tmem_base;

  // Register re-split: 384 threads x 168 registers are allocated at launch; the producer warpgroup
  // drops to 40 and the two epilogue warpgroups rise to 232 (128*40 + 256*232 = 384*168 exactly --
  // a larger request would wait forever for registers that are never released).
  static_assert(128 * 40 + 256 * 232 <= kNumThreads * 168, "setmaxnreg split exceeds the launch allocation");
  if (warp < 4) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 40;");
    if (warp == 0 && lane == 0) {
      // ---------------------------------------------------------------- TMA producer
      int stage = 0;
      uint32_t phase = 0;
      const uint32_t tx_bytes = (gather ? 0u : uint32_t(a.tile_m) * BK) + kBTileBytes;
      bool ok = true;
      PROF_DECL
      int mb_next = 0, n_next = 0, e_next = -1;
      if (int(blockIdx.x) < sched.total) {
        sched.decode(blockIdx.x, mb_next, n_next);
        e_next = __ldg(a.sorted_expert_ids + mb_next);
      }
      for (int t = blockIdx.x; t < sched.total && ok; t += gridDim.x) {
        const int mb = mb_next, n = n_next, e = e_next;
        if (t + int(gridDim.x) < sched.total) {          // next tile's expert id: loaded a whole tile early
          sched.decode(t + gridDim.x, mb_next, n_next);
          e_next = __ldg(a.sorted_expert_ids + mb_next);
        }
        if (e < 0 || e >= a.experts) continue;
        for (int kb = 0; kb < KB; ++kb) {
          PROF_START
          if (!mbar_wait(smem_u32(&ctrl->empty[stage]), phase ^ 1, abort_flag, a.status, 1, 64)) { ok = false; break; }
          PROF_STOP(0) PROF_COUNT(5)
          const uint32_t full = smem_u32(&ctrl->full[stage]);
          const uint32_t sa = smem_u32(smem + size_t(stage) * kStageBytes);
          const uint32_t sb = sa + kATileBytes;
          mbar_expect_tx(full, tx_bytes);
          if (!gather) tma_load_2d(sa, &tmap_a, full, kb * BK, mb * a.tile_m);
          if (STAGE == 1) {
            tma_load_3d(sb, &tmap_b, full, kb * BK, n * 128, e);
            tma_load_3d(sb + 128 * BK, &tmap_b, full, kb * BK, a.n_dim + n * 128, e);
          } else {
            tma_load_3d(sb, &tmap_b, full, kb * BK, n * BN, e);
          }
          if (++stage == kStages) { stage = 0; phase ^= 1; }
        }
      }
      PROF_WRITE(0);
    } else if (warp == 1 && lane == 0) {
      // ---------------------------------------------------------------- MMA issuer
      int stage = 0, acc = 0;
      uint32_t phase = 0, acc_phase = 0;
      bool ok = true;
      PROF_DECL
      const bool int8_ops = SCALING == kScalePerToken && a.in_dtype == FLYMOE_I8;
      const bool half_ops = SCALING == kScalePerToken && (a.in_dtype == FLYMOE_F16 || a.in_dtype == FLYMOE_BF16);
      const uint32_t half_desc = a.in_dtype == FLYMOE_BF16 ? kInstrDescBF16 : kInstrDescF16;
      int mb_next = 0, n_next = 0, e_next = -1;
      if (int(blockIdx.x) < sched.total) {
        sched.decode(blockIdx.x, mb_next, n_next);
        e_next = __ldg(a.sorted_expert_ids + mb_next);
      }
      for (int t = blockIdx.x; t < sched.total && ok; t += gridDim.x) {
        const int e = e_next;
        if (t + int(gridDim.x) < sched.total) {
          sched.decode(t + gridDim.x, mb_next, n_next);
          e_next = __ldg(a.sorted_expert_ids + mb_next);
        }
        if (e < 0 || e >= a.experts) continue;
        if (SCALING == kScalePerToken) {       // one accumulator stage per tile
          PROF_START
          if (!mbar_wait(smem_u32(&ctrl->tmem_empty[acc]), acc_phase ^ 1, abort_flag, a.status, 2)) { ok = false; break; }
          PROF_STOP(0)
        }
        for (int kb = 0; kb < KB; ++kb) {
          if (SCALING == kScaleBlock128) {     // one accumulator stage per K block, started from zero
            PROF_START
            if (!mbar_wait(smem_u32(&ctrl->tmem_empty[acc]), acc_phase ^ 1, abort_flag, a.status, 2)) { ok = false; break; }
            PROF_STOP(0)
          }
          PROF_START
          if (!mbar_wait(smem_u32(&ctrl->full[stage]), phase, abort_flag, a.status, 3)) { ok = false; break; }
          PROF_STOP(1)
          PROF_COUNT(5) PROF_START
          tcgen05_fence_after();
          const uint32_t sa = smem_u32(smem + size_t(stage) * kStageBytes);
          const uint64_t adesc = make_smem_desc(sa);
          const uint64_t bdesc = make_smem_desc(sa + kATileBytes);
          const uint32_t d_tmem = tmem_base + uint32_t(acc) * BN;
#pragma unroll
          for (int k = 0; k < BK / 32; ++k) {
            const uint32_t accumulate = (k > 0 || (SCALING == kScalePerToken && kb > 0)) ? 1u : 0u;
            if (int8_ops) umma_i8(d_tmem, adesc + uint64_t(k * 2), bdesc + uint64_t(k * 2), kInstrDescI8, accumulate);
            else if (half_ops) umma_f16(d_tmem, adesc + uint64_t(k * 2), bdesc + uint64_t(k * 2), half_desc, accumulate);
            else umma_f8(d_tmem, adesc + uint64_t(k * 2), bdesc + uint64_t(k * 2), kInstrDescF8, accumulate);
          }
          umma_commit(smem_u32(&ctrl->empty[stage]));
          if (SCALING == kScaleBlock128 || kb + 1 == KB) {
            umma_commit(smem_u32(&ctrl->tmem_full[acc]));
            if (++acc == kAccStages) { acc = 0; acc_phase ^= 1; }
          }
          PROF_STOP(3)
          if (++stage == kStages) { stage = 0; phase ^= 1; }
        }
      }
      PROF_WRITE(1);
    } else if (warp == 2 && uses_staging) {
      // ---------------------------------------------------------------- store warp
      // Issues the bulk store / bulk reduce of every epilogue thread's staging slot, eight slots per
      // lane, so that the ~10 cycles each of those 256 operations takes to be accepted are spent here
      // and not by the epilogue warps between two tiles.
      bool ok = true;
      uint32_t it = 0;
      int mb_next = 0, n_next = 0, e_next = -1;
      if (int(blockIdx.x) < sched.total) {
        sched.decode(blockIdx.x, mb_next, n_next);
        e_next = __ldg(a.sorted_expert_ids + mb_next);
      }
      constexpr uint32_t kSlotBytes = STAGE == 1 ? 64u : 256u;
      const bool bf = a.out_dtype == FLYMOE_BF16;
      for (int t = blockIdx.x; t < sched.total && ok; t += gridDim.x) {
        const int e = e_next, n = n_next;
        if (t + int(gridDim.x) < sched.total) {
          sched.decode(t + gridDim.x, mb_next, n_next);
          e_next = __ldg(a.sorted_expert_ids + mb_next);
        }
        if (e < 0 || e >= a.experts) continue;
        if (!mbar_wait(smem_u32(&ctrl->stg_full), it & 1, abort_flag, a.status, 6, 64)) { ok = false; break; }
        // stage 2 with n_dim = 64 mod 128 (dense GEMM only): the tile's last segment holds 64 columns
        const int cols_left = STAGE == 2 ? a.n_dim - n * BN : 0;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const int sl = i * 32 + lane;
          const unsigned long long dst = ctrl->stg_dst[sl];
          if (dst != 0ull) {
            const uint32_t sp = smem_u32(staging + size_t(sl) * Staging<STAGE>::stride);
            void* gp = reinterpret_cast<void*>(dst);
            const uint32_t bytes = (STAGE == 2 && cols_left - (sl >> 7) * 128 < 128) ? kSlotBytes / 2 : kSlotBytes;
            if (STAGE == 1 || !a.accumulate) bulk_store(gp, sp, bytes);
            else if (bf) bulk_reduce_add_bf16(gp, sp, bytes);
            else bulk_reduce_add_f16(gp, sp, bytes);
          }
        }
        asm volatile("cp.async.bulk.commit_group;" ::: "memory");
        bulk_wait_read_all();                      // the slots may be overwritten from here on
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&ctrl->stg_free));
        ++it;
      }
      bulk_wait_all();                             // every row segment has landed before the CTA retires
    } else if (warp == 3 && gather) {
      // ---------------------------------------------------------------- row gather
      // Lane l serves rows l, l+32, l+64, l+96 of the tile: eight 16-byte cp.async per row and K block,
      // written where the 128-byte swizzle puts them (chunk c of row r at r*128 + ((c ^ (r & 7)) << 4)).
      // A K block's copies are completed two K blocks later (cp.async.wait_group), made visible to the
      // tensor cores' proxy (fence.proxy.async) and then signalled on the stage's full barrier, next to
      // the TMA thread's arrival for the weights.  Pad rows are zero-filled (source size 0).
      // One warp issues every request, which keeps up with row blocks of 16 or 32 rows (decode); for
      // 64 and 128 rows it is slower than gathering ahead of the launch (measured: stage 1 of the
      // T=4096 layer 2.5 ms against 1.9 + 0.08 ms), so the host wrappers gather ahead for those.
      constexpr int kInFlight = 2;
      int stage = 0, pending = 0;
      uint32_t phase = 0;
      bool ok = true;
      const int pad_id = (a.topk << 24) | a.num_tokens;
      auto complete_oldest = [&]() {             // the oldest pending K block's rows have landed
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncwarp();
        const int s_old = (stage - pending + 2 * kStages) % kStages;
        if (lane == 0) mbar_arrive(smem_u32(&ctrl->full[s_old]));
        --pending;
      };
      for (int t = blockIdx.x; t < sched.total && ok; t += gridDim.x) {
        int mb, n;
        sched.decode(t, mb, n);
        const int e = __ldg(a.sorted_expert_ids + mb);
        if (e < 0 || e >= a.experts) continue;
        const uint8_t* src[4];
        uint32_t nbytes[4];                      // 16 = copy, 0 = zero-fill (pad row)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int row = j * 32 + lane;
          const int r = mb * a.tile_m + row;
          const int id = (row < a.tile_m && r < valid_rows) ? __ldg(a.sorted_ids + r) : pad_id;
          const int tok = id_token(id), slot = id_slot(id);
          const bool valid = tok < a.num_tokens && slot < a.topk;
          const long long srow = a.a_layout == FLYMOE_ROWS_BY_TOKEN ? (long long)tok
                               : a.a_layout == FLYMOE_ROWS_BY_SLOT ? (long long)slot * a.num_tokens + tok
                                                                   : (long long)tok * a.topk + slot;
          src[j] = a.a + (valid ? srow : 0) * a.k_dim;
          nbytes[j] = valid ? 16u : 0u;
        }
        for (int kb = 0; kb < KB; ++kb) {
          if (!mbar_wait(smem_u32(&ctrl->empty[stage]), phase ^ 1, abort_flag, a.status, 10, 32)) { ok = false; break; }
          const uint32_t sa = smem_u32(smem + size_t(stage) * kStageBytes);
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const int row = j * 32 + lane;
            if (row < a.tile_m) {
              const uint8_t* g = src[j] + kb * BK;
              const uint32_t d = sa + uint32_t(row) * 128u;
#pragma unroll
              for (int c = 0; c < 8; ++c)
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;"
                             ::"r"(d + (uint32_t(c ^ (row & 7)) << 4)), "l"(g + c * 16), "r"(nbytes[j]) : "memory");
            }
          }
          asm volatile("cp.async.commit_group;" ::: "memory");
          if (++stage == kStages) { stage = 0; phase ^= 1; }
          if (++pending > kInFlight) {
            asm volatile("cp.async.wait_group %0;" ::"n"(kInFlight) : "memory");
            complete_oldest();
          }
        }
      }
      asm volatile("cp.async.wait_group 0;" ::: "memory");
      while (pending > 0) complete_oldest();
    }
  } else {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 232;");
    // ------------------------------------------------------------------ epilogue
    const int wg = (warp - 4) >> 2;          // 0 or 1
    const int q = warp & 3;                  // TMEM lane quadrant of this warp
    const int row_in_tile = q * 32 + lane;
    const bool warp_active = q * 32 < a.tile_m;
    const uint32_t lane_base = uint32_t(q * 32) << 16;
    int acc = 0;
    uint32_t acc_phase = 0;
    uint32_t tile_iter = 0;
    bool ok = true;
    PROF_DECL
    static_assert(kAccStages == 2, "the epilogue's stage/phase stepping assumes two accumulator stages");
    const uint32_t full_bar0 = smem_u32(&ctrl->tmem_full[0]);     // stage 1's barrier is 8 bytes further
    const uint32_t empty_bar0 = smem_u32(&ctrl->tmem_empty[0]);
    constexpr int NACC = 128;                // fp32 accumulators per thread
    // Routing of a tile (expert id, this thread's packed row id) is loaded one tile ahead.
    const int pad_id = (a.topk << 24) | a.num_tokens;
    int mb_next = 0, n_next = 0, e_next = -1, id_next = pad_id;
    auto load_routing = [&](int tt) {
      sched.decode(tt, mb_next, n_next);
      e_next = __ldg(a.sorted_expert_ids + mb_next);
      const int rr = mb_next * a.tile_m + row_in_tile;
      id_next = (row_in_tile < a.tile_m && rr < valid_rows) ? __ldg(a.sorted_ids + rr) : pad_id;
    };
    if (int(blockIdx.x) < sched.total) load_routing(blockIdx.x);
    for (int t = blockIdx.x; t < sched.total && ok; t += gridDim.x) {
      const int mb = mb_next, n = n_next, e = e_next, id = id_next;
      if (t + int(gridDim.x) < sched.total) load_routing(t + gridDim.x);
      if (e < 0 || e >= a.experts) continue;

      const int r = mb * a.tile_m + row_in_tile;
      const bool in_tile = row_in_tile < a.tile_m && r < valid_rows;
      const int tok = id_token(id), slot = id_slot(id);
      const bool valid = in_tile && tok < a.num_tokens && slot < a.topk;
      long long sidx = 0;
      if (valid) {
        sidx = a.a_scale_layout == FLYMOE_ROWS_BY_TOKEN ? (long long)tok
             : a.a_scale_layout == FLYMOE_ROWS_BY_PAIR ? (long long)tok * a.topk + slot : (long long)r;
        if (SCALING == kScalePerToken && a.a_scale_layout == FLYMOE_ROWS_BY_SLOT) sidx = (long long)slot * a.num_tokens + tok;
      }
      // stage 2: a warpgroup whose 128 columns lie beyond n_dim (last tile of a row) has nothing to do
      const bool half_ok = STAGE == 1 ? true : (n * BN + wg * 128 < a.n_dim);
      // routing weight of this row, used after the K loop.  The loop runs at the register limit, and where
      // this value is requested decides whether ptxas spills inside it: stage 2 asks here (its latency
      // hides behind the loop), stage 1 after the loop (measured: no spills either way, `-Xptxas -v`).
      float wgt = 1.f;
      if (STAGE == 2 && a.doweight && valid) wgt = __ldg(a.sorted_weights + r);
      const bool work = warp_active && half_ok;
      // stage 1: first half = gate columns, second half = up columns; stage 2: two halves of 128 columns
      const uint32_t tcol0 = tmem_base + lane_base + (STAGE == 1 ? uint32_t(wg * 64) : uint32_t(wg * 128));
      const uint32_t tcol1 = tmem_base + lane_base + (STAGE == 1 ? uint32_t(128 + wg * 64) : uint32_t(wg * 128 + 64));
      float accv[NACC];
      if (SCALING == kScaleBlock128) {
      const float* sa_ptr = a.scale_a + sidx * a.sa_row_stride;
      // weight block scales of this tile
      const int wblk_per_expert = (STAGE == 1 ? 2 * a.n_dim : a.n_dim) / 128;
      const int blk0 = STAGE == 1 ? n : n * 2 + wg;
      const int blk1 = STAGE == 1 ? a.n_dim / 128 + n : blk0;
      const float* sw0_ptr = a.scale_w + ((long long)e * wblk_per_expert + (half_ok ? blk0 : 0)) * KB;
      const int sw1_off = (blk1 - (half_ok ? blk0 : 0)) * KB;      // up-projection scales, relative to sw0_ptr

      // fp32 accumulators held as packed pairs so the scale-FMA runs as fma.rn.f32x2
      unsigned long long acc2[NACC / 2];
#pragma unroll
      for (int j = 0; j < NACC / 2; ++j) acc2[j] = 0ull;

      float sa_next = valid ? __ldg(sa_ptr) : 0.f;
      float s0_next = __ldg(sw0_ptr);
      float s1_next = STAGE == 1 ? __ldg(sw0_ptr + sw1_off) : 0.f;
      const float* sa_run = sa_ptr;            // running pointer: one add per K block, no multiply
      // One K block = four 32-column chunks through two register buffers, two tcgen05.ld in flight at
      // a time: the thread waits twice per K block, not once per chunk.
      uint32_t v0[32], v1[32];
      // measured: two K blocks per loop trip help stage 1 (~1.5 %) and cost stage 2 about as much
#pragma unroll (STAGE == 1 ? 2 : 1)
      for (int kb = 0; kb < KB; ++kb) {
        const uint32_t stage_off = uint32_t(acc) * BN;
        PROF_START
        if (!mbar_wait(full_bar0 + uint32_t(acc) * 8u, acc_phase, abort_flag, a.status, 4)) { ok = false; break; }
        PROF_STOP(0) PROF_COUNT(5)
        tcgen05_fence_after();
        if (work) {                            // both chunks of the first half on their way at once
          tmem_ld_x32(tcol0 + stage_off, v0);
          tmem_ld_x32(tcol0 + stage_off + 32, v1);
        }
        const unsigned long long c0 = pack_f32x2(sa_next * s0_next);
        const unsigned long long c1 = STAGE == 1 ? pack_f32x2(sa_next * s1_next) : c0;
        if (work) tmem_ld_wait();
        if (kb + 1 < KB) {                     // next K block's scales: in flight during this block's math
          sa_run += a.sa_stride;
          sa_next = valid ? __ldg(sa_run) : 0.f;
          s0_next = __ldg(sw0_ptr + kb + 1);
          if (STAGE == 1) s1_next = __ldg(sw0_ptr + kb + 1 + sw1_off);
        }
        if (work) {
          // each buffer is refilled with its chunk of the second half as soon as it has been folded in
#pragma unroll
          for (int j = 0; j < 16; ++j) ffma2(acc2[j], v0[2 * j], v0[2 * j + 1], c0);
          tmem_ld_x32(tcol1 + stage_off, v0);
#pragma unroll
          for (int j = 0; j < 16; ++j) ffma2(acc2[16 + j], v1[2 * j], v1[2 * j + 1], c0);
          tmem_ld_x32(tcol1 + stage_off + 32, v1);
          tmem_ld_wait();
        }
        // The K block's partial sums are in registers now (tcgen05.wait::ld has returned, so the loads
        // have completed and need no further ordering): hand the TMEM stage back before the last
        // chunk's FMAs.  The arrive publishes no memory, hence relaxed; tcgen05.wait::ld is warp-wide
        // (.sync.aligned), so when lane 0 is past it every lane's loads have landed.
        if (!work) __syncwarp();
        if (lane == 0) mbar_arrive_relaxed(empty_bar0 + uint32_t(acc) * 8u);
        if (work) {
#pragma unroll
          for (int j = 0; j < 16; ++j) ffma2(acc2[32 + j], v0[2 * j], v0[2 * j + 1], c1);
#pragma unroll
          for (int j = 0; j < 16; ++j) ffma2(acc2[48 + j], v1[2 * j], v1[2 * j + 1], c1);
        }
        acc_phase ^= uint32_t(acc);
        acc ^= 1;
      }
      if (!ok) break;
#pragma unroll
      for (int j = 0; j < NACC / 2; ++j) unpack_f32x2(acc2[j], accv[2 * j], accv[2 * j + 1]);
      } else {
        // One scale per activation row, one per weight row: the whole K range has been accumulated in
        // TMEM; drain the tile once and scale it here.
        const uint32_t stage_off = uint32_t(acc) * BN;
        PROF_START
        if (!mbar_wait(full_bar0 + uint32_t(acc) * 8u, acc_phase, abort_flag, a.status, 4)) { ok = false; break; }
        PROF_STOP(0) PROF_COUNT(5)
        tcgen05_fence_after();
        // the raw accumulators land in the registers of accv and are scaled in place
        uint32_t* v = reinterpret_cast<uint32_t*>(accv);
        if (work) {
          tmem_ld_x32(tcol0 + stage_off, v);
          tmem_ld_x32(tcol0 + stage_off + 32, v + 32);
          tmem_ld_x32(tcol1 + stage_off, v + 64);
          tmem_ld_x32(tcol1 + stage_off + 32, v + 96);
          tmem_ld_wait();
        } else {
          __syncwarp();
        }
        if (lane == 0) mbar_arrive_relaxed(empty_bar0 + uint32_t(acc) * 8u);
        acc_phase ^= uint32_t(acc);
        acc ^= 1;
        if (work) {
          // 16-bit operands come without scales (null pointers): every factor is 1
          const float sa = valid ? (a.scale_a ? __ldg(a.scale_a + sidx) : 1.f) : 0.f;
          const long long wrows = STAGE == 1 ? 2LL * a.n_dim : (long long)a.n_dim;
          // weight-row scales of this thread's two 64-column halves (the same addresses in every lane)
          const float* sw0 = a.scale_w + (long long)e * wrows + (STAGE == 1 ? n * 128 + wg * 64 : n * BN + wg * 128);
          const float* sw1 = STAGE == 1 ? sw0 + a.n_dim : sw0 + 64;
          const bool i8 = a.in_dtype == FLYMOE_I8;
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            const float* sw = h == 0 ? sw0 : sw1;
#pragma unroll
            for (int j = 0; j < 64; j += 4) {
              const float4 s4 = a.scale_w ? __ldg(reinterpret_cast<const float4*>(sw + j)) : make_float4(1.f, 1.f, 1.f, 1.f);
              const float c[4] = {s4.x, s4.y, s4.z, s4.w};
#pragma unroll
              for (int u = 0; u < 4; ++u) {
                const int idx = h * 64 + j + u;
                const float p = i8 ? __int2float_rn(int(v[idx])) : accv[idx];
                accv[idx] = p * (sa * c[u]);
              }
              asm volatile("" ::: "memory");       // keeps the 32 scale loads from being hoisted in front of the math
            }
          }
        } else {
#pragma unroll
          for (int j = 0; j < NACC; ++j) accv[j] = 0.f;
        }
      }
      // Destination of this row when the caller gave per-row addresses: requested after the K loop (the
      // loop runs at the register limit) and needed only once the row has been packed.
      unsigned long long row_dst_base = 0ull;
      if (STAGE == 2 && ROW_DST && valid)
        row_dst_base = __ldg(a.row_dst + ((long long)tok * a.topk + slot));
      if (STAGE == 1 && a.doweight && valid) wgt = __ldg(a.sorted_weights + r);

      // ---- tile epilogue -----------------------------------------------------------
      // Kept short on purpose: this code runs once per tile between two main loops, and a long
      // straight-line tail (IEEE division, accurate exp) costs more in instruction fetch than in math.
      PROF_START
      if (STAGE == 1 && SCALING == kScalePerToken && a.out_dtype == FLYMOE_F32) {
        // The reference's split-K output contract (kernels/moe_gemm_2stage.py:121-122, :1345): the scaled gate
        // and up sums are ADDED to out[t*topk+s][0:I | I:2I] (fp32, zeroed by the caller) -- no activation,
        // no routing weight.  The whole K range is summed here, so every element receives one addition.
        if (warp_active && valid) {
          float* og = static_cast<float*>(a.out) + ((long long)tok * a.topk + slot) * (2LL * a.n_dim) +
                      (long long)n * 128 + wg * 64;
          float* ou = og + a.n_dim;
#pragma unroll
          for (int j = 0; j < 64; j += 4) red_add_v4_f32(og + j, accv[j], accv[j + 1], accv[j + 2], accv[j + 3]);
#pragma unroll
          for (int j = 0; j < 64; j += 4)
            red_add_v4_f32(ou + j, accv[64 + j], accv[64 + j + 1], accv[64 + j + 2], accv[64 + j + 3]);
        }
      } else if (STAGE == 1) {
        // accv[0..63] = gate, accv[64..127] = up, columns n*128 + wg*64 + j
        float amax = 0.f;
#pragma unroll
        for (int j = 0; j < 64; ++j) {
          const float g = accv[j];
          const float hval = g * fast_rcp(1.0f + fast_exp2(-1.4426950408889634f * g)) * (accv[64 + j] * wgt);
          accv[j] = hval;
          amax = fmaxf(amax, fabsf(hval));
        }
        const long long orow = a.out_layout == FLYMOE_ROWS_SORTED ? (long long)r : (long long)tok * a.topk + slot;
        const long long ocol = (long long)n * 128 + wg * 64;
        if (a.out_dtype == FLYMOE_E4M3) {
          const int buf = tile_iter & 1;
          const uint32_t bar = smem_u32(&ctrl->amax_bar[buf]);
          if (warp_active) ctrl->amax[buf][wg][row_in_tile] = valid ? amax : 0.f;
          __syncwarp();
          if (lane == 0) mbar_arrive(bar);
          if (!mbar_wait(bar, (tile_iter >> 1) & 1, abort_flag, a.status, 5)) { ok = false; break; }
          // the store warp has finished reading the previous tile's slots
          if (!mbar_wait(smem_u32(&ctrl->stg_free), (tile_iter & 1) ^ 1, abort_flag, a.status, 7)) { ok = false; break; }
          unsigned long long dst_addr = 0ull;
          const bool wr = warp_active && (valid || (in_tile && a.out_layout == FLYMOE_ROWS_SORTED));
          if (wr) {
            const float m = fmaxf(ctrl->amax[buf][0][row_in_tile], ctrl->amax[buf][1][row_in_tile]);
            float sc = __fdiv_rn(m, 448.0f);
            if (sc == 0.f) sc = 1.f;
            const float inv = valid ? __fdiv_rn(1.0f, sc) : 0.f;     // pad rows: every code becomes 0
            // 64 codes go through this thread's staging slot and leave as one 64-byte bulk store
            uint8_t* op = staging + size_t(threadIdx.x - 128) * Staging<STAGE>::stride;
#pragma unroll
            for (int j = 0; j < 64; j += 16) {
              uint4 pk;
              pk.x = float4_to_e4m3x4(accv[j + 0] * inv, accv[j + 1] * inv, accv[j + 2] * inv, accv[j + 3] * inv);
              pk.y = float4_to_e4m3x4(accv[j + 4] * inv, accv[j + 5] * inv, accv[j + 6] * inv, accv[j + 7] * inv);
              pk.z = float4_to_e4m3x4(accv[j + 8] * inv, accv[j + 9] * inv, accv[j + 10] * inv, accv[j + 11] * inv);
              pk.w = float4_to_e4m3x4(accv[j + 12] * inv, accv[j + 13] * inv, accv[j + 14] * inv, accv[j + 15] * inv);
              if (!valid) pk = make_uint4(0, 0, 0, 0);
              *reinterpret_cast<uint4*>(op + j) = pk;
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            dst_addr = reinterpret_cast<unsigned long long>(static_cast<uint8_t*>(a.out) + orow * a.n_dim + ocol);
            if (wg == 0) a.out_scale[(long long)n * a.out_scale_stride + orow] = sc;
          }
          ctrl->stg_dst[threadIdx.x - 128] = dst_addr;
          __syncwarp();
          if (lane == 0) mbar_arrive(smem_u32(&ctrl->stg_full));
        } else if (warp_active && valid) {
          uint8_t* op = static_cast<uint8_t*>(a.out) + (orow * a.n_dim + ocol) * 2;
          const bool bf = a.out_dtype == FLYMOE_BF16;
#pragma unroll
          for (int j = 0; j < 64; j += 8) {
            uint4 pk;
            pk.x = bf ? pack_bf16x2(accv[j + 0], accv[j + 1]) : pack_f16x2(accv[j + 0], accv[j + 1]);
            pk.y = bf ? pack_bf16x2(accv[j + 2], accv[j + 3]) : pack_f16x2(accv[j + 2], accv[j + 3]);
            pk.z = bf ? pack_bf16x2(accv[j + 4], accv[j + 5]) : pack_f16x2(accv[j + 4], accv[j + 5]);
            pk.w = bf ? pack_bf16x2(accv[j + 6], accv[j + 7]) : pack_f16x2(accv[j + 6], accv[j + 7]);
            *reinterpret_cast<uint4*>(op + j * 2) = pk;
          }
        }
      } else if (a.out_dtype == FLYMOE_F32) {
        if (warp_active && valid && half_ok) {
          // fp32 output: vector reductions straight from registers (accumulate mode only)
          float* op = static_cast<float*>(a.out) + (long long)tok * a.n_dim + (long long)n * BN + wg * 128;
#pragma unroll
          for (int j = 0; j < 128; j += 4)
            red_add_v4_f32(op + j, accv[j] * wgt, accv[j + 1] * wgt, accv[j + 2] * wgt, accv[j + 3] * wgt);
        }
      } else {
        // 16-bit output: each thread parks its 128 results (256 B) in its own slot of the staging area
        // together with the global address of its row segment; the store warp sends every slot off as
        // ONE bulk reduce-add (or bulk store), instead of 16 scattered 16-byte atomics per thread.
        uint8_t* slot_ptr = staging + size_t(threadIdx.x - 128) * Staging<STAGE>::stride;
        if (!mbar_wait(smem_u32(&ctrl->stg_free), (tile_iter & 1) ^ 1, abort_flag, a.status, 7)) { ok = false; break; }
        unsigned long long dst_addr = 0ull;
        if (warp_active && valid && half_ok) {
          const bool bf = a.out_dtype == FLYMOE_BF16;
#pragma unroll
          for (int j = 0; j < 128; j += 8) {
            uint4 pk;
            pk.x = bf ? pack_bf16x2(accv[j] * wgt, accv[j + 1] * wgt) : pack_f16x2(accv[j] * wgt, accv[j + 1] * wgt);
            pk.y = bf ? pack_bf16x2(accv[j + 2] * wgt, accv[j + 3] * wgt) : pack_f16x2(accv[j + 2] * wgt, accv[j + 3] * wgt);
            pk.z = bf ? pack_bf16x2(accv[j + 4] * wgt, accv[j + 5] * wgt) : pack_f16x2(accv[j + 4] * wgt, accv[j + 5] * wgt);
            pk.w = bf ? pack_bf16x2(accv[j + 6] * wgt, accv[j + 7] * wgt) : pack_f16x2(accv[j + 6] * wgt, accv[j + 7] * wgt);
            *reinterpret_cast<uint4*>(slot_ptr + j * 2) = pk;
          }
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
          const long long orow = a.accumulate ? (long long)tok : (long long)tok * a.topk + slot;
          const long long col_bytes = ((long long)n * BN + wg * 128) * 2;
          if (ROW_DST) {
            // rows leave for caller-given addresses (another GPU's buffer included): the bulk store
            // carries the row segment there while the next tile is in the tensor cores
            // a misaligned address would fault the bulk store: drop the row and report instead
            const unsigned long long base = row_dst_base;
            if ((base & 15ull) != 0ull) atomicCAS(a.status, 0, FLYMOE_STATUS_ROW_DST_MISALIGNED);
            else dst_addr = base != 0ull ? base + (unsigned long long)col_bytes : 0ull;
          } else {
            dst_addr = reinterpret_cast<unsigned long long>(static_cast<uint8_t*>(a.out) + orow * a.n_dim * 2 + col_bytes);
          }
        }
        ctrl->stg_dst[threadIdx.x - 128] = dst_addr;
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&ctrl->stg_full));
      }
      PROF_STOP(1) PROF_COUNT(4)
      ++tile_iter;
    }
    if (threadIdx.x == 128) PROF_WRITE(2);
  }

  tcgen05_fence_before();
  __syncthreads();
  if (warp == 1) {
    tcgen05_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(uint32_t(kTmemCols))
                 : "memory");
  }
}

// One thread waits, with the kernels' own bounded wait, on a barrier that nobody arrives at.
__global__ void bounded_wait_selftest_kernel(int* status, unsigned long long limit_ns, int code) {
  __shared__ unsigned long long bar;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    mbar_init(smem_u32(&bar), 1);
    abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  if (threadIdx.x == 0) mbar_wait(smem_u32(&bar), 0, &abort_flag, status, code, 64, limit_ns);
}

}  // namespace flymoe

extern "C" int flymoe_set_gemm_cta_limit(int max_ctas) {
  if (max_ctas < 0) {
    flymoe::set_last_error_msg("set_gemm_cta_limit: max_ctas must be >= 0");
    return FLYMOE_ERR_INVALID_ARGUMENT;
  }
  flymoe::g_cta_limit = max_ctas;
  return FLYMOE_OK;
}

extern "C" int flymoe_selftest_bounded_wait(int64_t limit_ns, void* stream) {
  using namespace flymoe;
  FLYMOE_REQUIRE(limit_ns > 0 && limit_ns <= 100000000, "selftest_bounded_wait: limit_ns must be in (0, 1e8]");
  int* status = device_status_ptr();
  FLYMOE_REQUIRE(status != nullptr, "selftest_bounded_wait: no CUDA device");
  bounded_wait_selftest_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(
      status, static_cast<unsigned long long>(limit_ns), FLYMOE_STATUS_SELFTEST_TIMEOUT);
  FLYMOE_CUDA_CHECK(cudaGetLastError());
  return FLYMOE_OK;
}

#ifdef FLYMOE_PROF
extern "C" int flymoe_prof_read(long long* host_out) {
  FLYMOE_CUDA_CHECK(cudaDeviceSynchronize());
  FLYMOE_CUDA_CHECK(cudaMemcpyFromSymbol(host_out, flymoe::g_prof, sizeof(flymoe::g_prof)));
  return FLYMOE_OK;
}
#endif

namespace flymoe {

// ------------------------------------------------------------------------------ host
static PFN_cuTensorMapEncodeTiled_v12000 encode_fn() {
  static PFN_cuTensorMapEncodeTiled_v12000 fn = nullptr;
  if (fn == nullptr) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPointByVersion("cuTensorMapEncodeTiled", &p, 12000, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(p);
  }
  return fn;
}

static int make_map(CUtensorMap* map, const void* base, int rank, const cuuint64_t* dims, const cuuint64_t* strides,
                    const cuuint32_t* box) {
  PFN_cuTensorMapEncodeTiled_v12000 fn = encode_fn();
  if (fn == nullptr) {
    set_last_error_msg("cuTensorMapEncodeTiled is not available from this driver");
    return FLYMOE_ERR_CUDA;
  }
  cuuint32_t elem_strides[3] = {1, 1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, rank, const_cast<void*>(base), dims, strides, box, elem_strides,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    char buf[128];
    snprintf(buf, sizeof(buf), "cuTensorMapEncodeTiled failed with CUresult %d", int(r));
    set_last_error_msg(buf);
    return FLYMOE_ERR_CUDA;
  }
  return FLYMOE_OK;
}

template <int STAGE, bool ROW_DST, int SCALING, bool GATHER>
static int launch_kernel(int grid, cudaStream_t stream, const CUtensorMap& map_a, const CUtensorMap& map_b,
                         const GemmArgs& a, int group_m) {
  auto* kernel = moe_gemm_sm100_kernel<STAGE, ROW_DST, SCALING, GATHER>;
  FLYMOE_CUDA_CHECK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         int(smem_bytes<STAGE>())));
  kernel<<<grid, kNumThreads, smem_bytes<STAGE>(), stream>>>(map_a, map_b, a, group_m);
  FLYMOE_CUDA_CHECK(cudaGetLastError());
  return FLYMOE_OK;
}

template <int STAGE, bool ROW_DST, int SCALING>
static int launch_one(int grid, cudaStream_t stream, const CUtensorMap& map_a, const CUtensorMap& map_b,
                      const GemmArgs& a, int group_m) {
  if (a.a_layout != FLYMOE_ROWS_SORTED)
    return launch_kernel<STAGE, ROW_DST, SCALING, true>(grid, stream, map_a, map_b, a, group_m);
  return launch_kernel<STAGE, ROW_DST, SCALING, false>(grid, stream, map_a, map_b, a, group_m);
}

int launch_gemm_sm100(int stage, const GemmArgs& a, cudaStream_t stream) {
  if (a.tile_m != 16 && a.tile_m != 32 && a.tile_m != 64 && a.tile_m != 128) {
    set_last_error_msg("tcgen05 GEMM: tile_m must be 16, 32, 64 or 128");
    return FLYMOE_ERR_UNSUPPORTED;
  }
  if (a.a_layout != FLYMOE_ROWS_SORTED && a.a_layout != FLYMOE_ROWS_BY_TOKEN && a.a_layout != FLYMOE_ROWS_BY_PAIR &&
      a.a_layout != FLYMOE_ROWS_BY_SLOT) {
    set_last_error_msg("tcgen05 GEMM: unknown activation row layout");
    return FLYMOE_ERR_UNSUPPORTED;
  }
  const bool per_token = a.scaling == FLYMOE_SCALE_PER_TOKEN;
  if (per_token && (a.row_dst != nullptr || a.out_dtype == FLYMOE_E4M3)) {
    set_last_error_msg("tcgen05 GEMM: per-token scaling supports neither per-row destinations nor e4m3 output");
    return FLYMOE_ERR_UNSUPPORTED;
  }
  const long long wrows = stage == 1 ? 2LL * a.n_dim : a.n_dim;
  CUtensorMap map_a, map_b;
  {
    cuuint64_t dims[2] = {cuuint64_t(a.k_dim), cuuint64_t(a.a_rows)};
    cuuint64_t strides[1] = {cuuint64_t(a.k_dim)};
    cuuint32_t box[2] = {cuuint32_t(BK), cuuint32_t(a.tile_m)};
    int rc = make_map(&map_a, a.a, 2, dims, strides, box);
    if (rc != FLYMOE_OK) return rc;
  }
  {
    cuuint64_t dims[3] = {cuuint64_t(a.k_dim), cuuint64_t(wrows), cuuint64_t(a.experts)};
    cuuint64_t strides[2] = {cuuint64_t(a.k_dim), cuuint64_t(wrows) * cuuint64_t(a.k_dim)};
    cuuint32_t box[3] = {cuuint32_t(BK), cuuint32_t(stage == 1 ? 128 : BN), 1};
    int rc = make_map(&map_b, a.w, 3, dims, strides, box);
    if (rc != FLYMOE_OK) return rc;
  }
  const long long pairs = (long long)a.num_tokens * a.topk;
  long long g = (pairs + (long long)a.experts * a.tile_m - 1) / ((long long)a.experts * a.tile_m);
  const int group_m = int(g < 1 ? 1 : (g > 16 ? 16 : g));
  const int ntiles = stage == 1 ? a.n_dim / 128 : ceil_div(a.n_dim, BN);
  const long long max_tiles = (long long)a.size_expert_ids * ntiles;
  int ctas = sm_count();
  if (g_cta_limit > 0 && g_cta_limit < ctas) ctas = g_cta_limit;
  const int grid = int(max_tiles < ctas ? max_tiles : ctas);
  if (grid <= 0) return FLYMOE_OK;
  if (per_token)
    return stage == 1 ? launch_one<1, false, kScalePerToken>(grid, stream, map_a, map_b, a, group_m)
                      : launch_one<2, false, kScalePerToken>(grid, stream, map_a, map_b, a, group_m);
  if (stage == 1) return launch_one<1, false, kScaleBlock128>(grid, stream, map_a, map_b, a, group_m);
  if (a.row_dst != nullptr) return launch_one<2, true, kScaleBlock128>(grid, stream, map_a, map_b, a, group_m);
  return launch_one<2, false, kScaleBlock128>(grid, stream, map_a, map_b, a, group_m);
}

}  // namespace flymoe
