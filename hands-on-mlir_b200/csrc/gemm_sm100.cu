// fp16 GEMM family for sm_100a: D = epilogue(alpha * A.B + beta * C), fp32 accumulate in
// tensor memory, Row,Row,Row operands (B as [K,N]) or the "transb" form (B as [N,K]).
//
// One persistent CTA per SM walks a static list of 128 x BN output tiles.  Inside a CTA:
//   warp 0    TMA producer: 128x64 A box + BN x 64 B boxes per K block into a ring of
//             128-byte-swizzled shared-memory stages (mbarrier full/empty hand-off);
//   warp 1    one thread issues tcgen05.mma (M=128, N=BN, K=16) into one of two TMEM
//             accumulators and releases stages / publishes accumulators with tcgen05.commit;
//   warps 2-9 epilogue (two warps per tensor-memory lane quarter, each a share of the tile's
//             columns): tcgen05.ld the finished accumulator (one output row per thread, 64
//             columns at a time), fp32 alpha/beta/bias/erf-GELU, one fp16 rounding, results
//             staged in swizzled shared memory and written out by TMA stores, while warp 1
//             already fills the other accumulator.
//
// This replaces the reference's CUTLASS 2.x mma.sync kernels and its compile-time autotuner
// (include/NVGPUKernels/GemmRunner.h:119-310, lib/NVGPUKernels/GemmProfiler.cu:143-236) with a
// small per-shape tile table.
#include <cstdlib>
#include <cstdio>
#include <tuple>
#include <map>
#include <cstring>
#include <mutex>
#include <unordered_map>

#include "gemm_epilogue.cuh"
#include "gemm_sm100.cuh"
#include "ptx_sm100.cuh"

namespace hom {
namespace gemm {

using namespace hom::ptx;

namespace {

constexpr int BM = 128;
constexpr int BK = 64;
constexpr int kThreads = 64 + 32 * kEpilogueWarps;
constexpr uint32_t kABytes = BM * BK * 2;

template <int BN>
struct TileCfg {
  static constexpr uint32_t kBBytes = BN * BK * 2;
  static constexpr uint32_t kStageBytes = kABytes + kBBytes;
  // As many stages as fit beside the 64 KB of epilogue staging.
  static constexpr int kStages = BN == 256 ? 3 : BN == 192 ? 4 : BN == 128 ? 5 : 6;
  static constexpr uint32_t kTmemCols = BN == 64 ? 128 : BN == 128 ? 256 : 512;
  static constexpr uint32_t kStagingBytes = kEpilogueStagingBytes;
  static constexpr uint32_t kBarrierBytes = 8 * (2 * kStages + 4) + 16;
  static constexpr uint32_t kSmemBytes = kStages * kStageBytes + kStagingBytes + kBarrierBytes + 1024;
};

struct Params {
  EpilogueParams ep;
  int K;
  int n_blocks, num_tiles, num_kb;
  int stages;  // ring slots in use, <= TileCfg::kStages
  int b_grouped;  // B [K,N] is fetched through the grouped 3-D tensor map (N % 64 == 0)
  int *status;
  long long *prof;  // optional per-role cycle counters of CTA 0 (diagnostics), else null
  long long *tl;    // optional launch-timeline slot (diagnostics), else null
  // fused LayerNorm over the output rows (LN kernels only): grid = tiles, one cluster per 128 rows
  float ln_eps, ln_inv_n;
  int ln_cluster;
};

// Wait that ignores the CTA abort flag; used only to let in-flight TMA land before exit.
__device__ __forceinline__ void mbar_wait_drain(uint32_t bar, uint32_t parity) {
  const long long t0 = clock64();
  while (!mbar_try_wait(bar, parity)) {
    if (clock64() - t0 > 200000000LL) break;
  }
}

template <int BN, bool B_NK, bool LN = false>
__global__ void __launch_bounds__(kThreads, 1)
gemm_f16_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                const __grid_constant__ CUtensorMap tmD, const Params p) {
  using Cfg = TileCfg<BN>;
  constexpr int STAGES = Cfg::kStages;  // ring slots laid out in shared memory
  const int stages_used = p.stages;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t smem_base = (raw_addr + 1023u) & ~1023u;
  uint8_t *smem_gen = smem_raw + (smem_base - raw_addr);

  const uint32_t staging_base = smem_base + STAGES * Cfg::kStageBytes;
  const uint32_t bar_base = staging_base + Cfg::kStagingBytes;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (STAGES + s); };
  auto tfull_bar = [&](int a) { return bar_base + 8u * (2 * STAGES + a); };
  auto tempty_bar = [&](int a) { return bar_base + 8u * (2 * STAGES + 2 + a); };
  volatile uint32_t *tmem_slot =
      reinterpret_cast<volatile uint32_t *>(smem_gen + STAGES * Cfg::kStageBytes + Cfg::kStagingBytes +
                                            8 * (2 * STAGES + 4));
  volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  const long long t_entry = p.prof ? clock64() : 0;
  unsigned long long g_entry = 0;
  if (p.prof) asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(g_entry));
  pdl_launch_dependents();
  if (p.tl && threadIdx.x == 0) timeline_stamp(p.tl, 0);
  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(tfull_bar(a), 1);
      mbar_init(tempty_bar(a), kEpilogueWarps);  // one arrival per epilogue warp
    }
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(const_cast<uint32_t *>(tmem_slot)), Cfg::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  if (p.prof && blockIdx.x == 0 && threadIdx.x == 0) p.prof[10] = clock64() - t_entry;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    // Run by the whole warp (coordinates and addresses stay warp-uniform); one elected lane
    // arms the barriers and issues the copies.
    {
      const bool leader = elect_one();
      if (leader) {
        prefetch_tensormap(&tmA);
        prefetch_tensormap(&tmB);
      }
      int s = 0;
      uint32_t ph = 0, armed = 0;
      bool ok = true;
      long long t_wait = 0, t_begin = clock64();
      auto load_b = [&](int slot, int kb, int n0) {
        const uint32_t b_dst = smem_base + slot * Cfg::kStageBytes + kABytes;
        if (!leader) return;
        if (B_NK) {
          tma_load_2d(b_dst, &tmB, full_bar(slot), kb * BK, n0);
        } else if (p.b_grouped) {
          tma_load_3d(b_dst, &tmB, full_bar(slot), 0, kb * BK, n0 / 64);
        } else {
#pragma unroll
          for (int g = 0; g < BN / 64; ++g)
            tma_load_2d(b_dst + g * (BK * 128), &tmB, full_bar(slot), n0 + g * 64, kb * BK);
        }
      };
      // B holds weights, which no earlier kernel of the stream writes: the first ring of B
      // tiles is requested before waiting for the previous kernel, A only after.
      int pre = 0;
      if (blockIdx.x < p.num_tiles) {
        const int n0 = (blockIdx.x % p.n_blocks) * BN;
        pre = p.num_kb < stages_used ? p.num_kb : stages_used;
        for (int kb = 0; kb < pre; ++kb) {
          if (leader) mbar_arrive_expect_tx(full_bar(kb), Cfg::kStageBytes);
          load_b(kb, kb, n0);
        }
      }
      pdl_wait();
      if (p.tl && leader) timeline_stamp(p.tl, 2);
      for (int tile = blockIdx.x; tile < p.num_tiles && ok; tile += gridDim.x) {
        const int m0 = (tile / p.n_blocks) * BM;
        const int n0 = (tile % p.n_blocks) * BN;
        for (int kb = 0; kb < p.num_kb; ++kb) {
          const bool b_done = tile == static_cast<int>(blockIdx.x) && kb < pre;
          if (!b_done) {
            const long long tw = p.prof ? clock64() : 0;
            ok = __all_sync(0xffffffffu, mbar_wait(empty_bar(s), ph ^ 1u, abort_flag, p.status,
                                                   kDevWaitTimeoutProducer));
            if (!ok) break;
            if (p.prof) t_wait += clock64() - tw;
            if (leader) mbar_arrive_expect_tx(full_bar(s), Cfg::kStageBytes);
            load_b(s, kb, n0);
          }
          if (leader) tma_load_2d(smem_base + s * Cfg::kStageBytes, &tmA, full_bar(s), kb * BK, m0);
          ++armed;
          if (++s == stages_used) {
            s = 0;
            ph ^= 1u;
          }
        }
      }
      if (p.prof && blockIdx.x == 0 && lane == 0) {
        p.prof[0] = clock64() - t_begin;
        p.prof[1] = t_wait;
      }
      if (!ok) {
        // Let every copy this warp started land before the CTA gives its shared memory back.
        for (int st = 0; st < stages_used; ++st) {
          const uint32_t n_st = armed / stages_used + (static_cast<uint32_t>(st) < armed % stages_used ? 1u : 0u);
          if (n_st > 0) mbar_wait_drain(full_bar(st), (n_st - 1u) & 1u);
        }
      }
      if constexpr (LN) cluster_sync_all();  // the epilogue's statistics exchange counts every thread
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------- MMA issuer
    // The whole warp runs the loop so that stage addresses and descriptors stay warp-uniform;
    // one elected lane issues the MMAs and the commits.
    {
      constexpr uint32_t idesc = make_idesc_f16(BM, BN, false, !B_NK);
      const bool leader = elect_one();
      int s = 0;
      uint32_t ph = 0;
      bool ok = true;
      int it = 0;
      long long t_full = 0, t_acc = 0, t_begin = clock64();
      for (int tile = blockIdx.x; tile < p.num_tiles && ok; tile += gridDim.x, ++it) {
        const int acc = it & 1;
        const uint32_t acc_ph = (it >> 1) & 1;
        const long long ta = p.prof ? clock64() : 0;
        ok = __all_sync(0xffffffffu,
                        mbar_wait(tempty_bar(acc), acc_ph ^ 1u, abort_flag, p.status, kDevWaitTimeoutMma));
        if (!ok) break;
        if (p.prof) t_acc += clock64() - ta;
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + acc * BN;
        bool have = false;  // full[s] already seen complete by the probe of the previous block
        for (int kb = 0; kb < p.num_kb; ++kb) {
          if (!have) {
            const long long tw = p.prof ? clock64() : 0;
            ok = __all_sync(0xffffffffu,
                            mbar_wait(full_bar(s), ph, abort_flag, p.status, kDevWaitTimeoutMma));
            if (!ok) break;
            if (p.prof) t_full += clock64() - tw;
          }
          have = false;
          tc_fence_after_sync();
          const uint32_t a_addr = smem_base + s * Cfg::kStageBytes;
          const uint32_t b_addr = a_addr + kABytes;
          const int s_next = s + 1 == stages_used ? 0 : s + 1;
          const uint32_t ph_next = s_next == 0 ? ph ^ 1u : ph;
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) {
            // A: K-major rows of 128 B; 8-row groups 1024 B apart; 16 K elements = 32 B.
            const uint64_t da = make_smem_desc_sw128(a_addr + k * 32, 16, 1024);
            // B as [N,K]: same as A.  B as [K,N] (N contiguous): 64-column groups are
            // separate sub-tiles BK*128 B apart, 8-row K groups 1024 B apart, and 16 K rows
            // = 2048 B.
            const uint64_t db = B_NK ? make_smem_desc_sw128(b_addr + k * 32, 16, 1024)
                                     : make_smem_desc_sw128(b_addr + k * 2048, BK * 128, 1024);
            if (leader) tc_mma_f16_ss(d_tmem, da, db, idesc, (kb | k) != 0 ? 1u : 0u);
            // Probe the next stage while the tensor pipe is busy with what was just queued.
            if (k == 1 && kb + 1 < p.num_kb)
              have = __all_sync(0xffffffffu, mbar_test_wait(full_bar(s_next), ph_next));
          }
          if (leader) tc_commit(empty_bar(s));
          s = s_next;
          ph = ph_next;
        }
        if (ok && leader) tc_commit(tfull_bar(acc));
      }
      if (p.prof && blockIdx.x == 0 && lane == 0) {
        p.prof[2] = clock64() - t_begin;
        p.prof[3] = t_full;
        p.prof[4] = t_acc;
      }
      if constexpr (LN) cluster_sync_all();  // the epilogue's statistics exchange counts every thread
    }
  } else {
    // --------------------------------------------------------------- epilogue
    const int quarter = warp & 3;       // TMEM lanes [32*quarter, 32*quarter + 32)
    const int group = (warp - 2) >> 2;  // which 64-column group of the tile
    const int col_begin = group * 64;
    const bool active = col_begin < BN;
    const uint32_t stage_smem = staging_base + (warp - 2) * kEpilogueStageBytes;
    int it = 0;
    bool ln_done = false;
    long long t_wait = 0, t_begin = clock64();
    pdl_wait();  // C may be produced, and D still read, by the previous kernel
    for (int tile = blockIdx.x; tile < p.num_tiles; tile += gridDim.x, ++it) {
      const int acc = it & 1;
      const uint32_t acc_ph = (it >> 1) & 1;
      const int m0 = (tile / p.n_blocks) * BM;
      const int n0 = (tile % p.n_blocks) * BN;
      uint4 cval[8];
      if (active) epilogue_load_c(p.ep, m0 + quarter * 32 + lane, n0 + col_begin, cval);
      const long long tw = p.prof ? clock64() : 0;
      bool ok = mbar_wait(tfull_bar(acc), acc_ph, abort_flag, p.status, kDevWaitTimeoutEpilogue);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      if (p.prof) t_wait += clock64() - tw;
      tc_fence_after_sync();
      const uint32_t t_row =
          tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + acc * BN + col_begin;
      if constexpr (LN) {
        // one tile per CTA; the pipeline stages are idle by now and stage 0 holds the statistics
        LayernormFusion ln;
        ln.stats_smem = smem_base;
        ln.cluster_n = p.ln_cluster;
        ln.row_in_tile = quarter * 32 + lane;
        ln.group = group;
        ln.eps = p.ln_eps;
        ln.inv_n = p.ln_inv_n;
        epilogue_warp_block_ln(p.ep, &tmD, t_row, m0 + quarter * 32, n0 + col_begin, active, stage_smem,
                               lane, cval, ln);
        ln_done = true;
      } else {
        epilogue_warp_block(p.ep, &tmD, t_row, m0 + quarter * 32, n0 + col_begin, active, stage_smem, lane,
                            cval, [&]() {
                              if (lane == 0) mbar_arrive(tempty_bar(acc));
                            });
      }
    }
    if constexpr (LN) {
      if (!ln_done) {  // error path: keep the named barrier's and the cluster barrier's counts whole
        asm volatile("bar.sync 1, 512;" ::: "memory");
        cluster_sync_all();
      }
    }
    // A store still in flight reads this warp's staging tile: let it finish reading.
    if (lane == 0) bulk_wait_group_read_0();
    __syncwarp();
    if (p.prof && blockIdx.x == 0 && threadIdx.x == 64) {
      p.prof[5] = clock64() - t_begin;
      p.prof[6] = t_wait;
    }
  }

  tc_fence_before_sync();
  if constexpr (LN) cluster_sync_all();  // peers may still be reading this CTA's statistics
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, Cfg::kTmemCols);
  }
  if (p.tl && threadIdx.x == 0) timeline_stamp(p.tl, 4);
  if (p.prof && blockIdx.x == 0 && threadIdx.x == 32) {
    unsigned long long g_exit;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(g_exit));
    p.prof[11] = clock64() - t_entry;
    p.prof[12] = static_cast<long long>(g_entry);
    p.prof[13] = static_cast<long long>(g_exit);
    // ring of (entry, exit) wall-clock stamps of the last launches (timeline diagnostics)
    const long long slot = p.prof[15] & 15;
    p.prof[16 + 2 * slot] = static_cast<long long>(g_entry);
    p.prof[17 + 2 * slot] = static_cast<long long>(g_exit);
    p.prof[15] += 1;
  }
}

// ------------------------------------------------------------------ host side

using EncodeFn = CUresult (*)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *,
                              const cuuint64_t *, const cuuint64_t *, const cuuint32_t *,
                              const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                              CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeFn get_encode_fn() {
  static EncodeFn fn = []() -> EncodeFn {
    void *sym = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPointByVersion("cuTensorMapEncodeTiled", &sym, 12000, cudaEnableDefault,
                                         &qres) != cudaSuccess ||
        qres != cudaDriverEntryPointSuccess)
      return nullptr;
    return reinterpret_cast<EncodeFn>(sym);
  }();
  return fn;
}

struct MapKey {
  const void *ptr;
  uint64_t inner, outer;
  uint32_t box_inner, box_outer;  // box_outer | groups << 16 for the grouped 3-D form
  bool operator==(const MapKey &o) const {
    return ptr == o.ptr && inner == o.inner && outer == o.outer && box_inner == o.box_inner &&
           box_outer == o.box_outer;
  }
};
struct MapKeyHash {
  size_t operator()(const MapKey &k) const {
    size_t h = reinterpret_cast<size_t>(k.ptr);
    h = h * 1000003u ^ k.inner;
    h = h * 1000003u ^ k.outer;
    h = h * 1000003u ^ (static_cast<size_t>(k.box_inner) << 16 | k.box_outer);
    return h;
  }
};

std::mutex g_map_mutex;
std::unordered_map<MapKey, CUtensorMap, MapKeyHash> g_map_cache;

}  // namespace

// Diagnostics (HOM_GEMM_PROFILE=1): a small device buffer the kernels fill with per-role
// cycle counters of CTA 0, printed after a stream synchronisation.  Never on by default.
static long long *g_profile_buf = nullptr;

long long *profile_buffer() {
  static bool checked = false;
  if (!checked) {
    checked = true;
    if (std::getenv("HOM_GEMM_PROFILE") || std::getenv("HOM_ATTN_PROFILE")) {
      if (cudaMalloc(&g_profile_buf, 4096 * sizeof(long long)) != cudaSuccess) g_profile_buf = nullptr;
      else {
        cudaMemset(g_profile_buf, 0, 4096 * sizeof(long long));
        // slots [32, 64): {first entry, last entry, first exit, last exit} of eight launches
        long long init[32];
        for (int i = 0; i < 32; ++i) init[i] = (i & 1) == 0 ? 0x7fffffffffffffffLL : 0;
        cudaMemcpy(g_profile_buf + 32, init, sizeof(init), cudaMemcpyHostToDevice);
        // slots [3800, 4088): {first, last} x {entry, dependency resolved, exit} of 48 GEMM launches
        long long init2[288];
        for (int i = 0; i < 288; ++i) init2[i] = (i & 1) == 0 ? 0x7fffffffffffffffLL : 0;
        cudaMemcpy(g_profile_buf + 3800, init2, sizeof(init2), cudaMemcpyHostToDevice);
      }
    }
  }
  // The role counters are only collected while one of the variables is (still) set, so that a
  // program can switch them off before it captures a graph.
  if (!g_profile_buf || !(std::getenv("HOM_GEMM_PROFILE") || std::getenv("HOM_ATTN_PROFILE"))) return nullptr;
  if (!std::getenv("HOM_GEMM_TIMELINE")) cudaMemset(g_profile_buf, 0, 15 * sizeof(long long));
  return g_profile_buf;
}

long long *profile_buffer_raw() { return g_profile_buf; }

// Launch timeline (HOM_GEMM_LAUNCH_TIMELINE set while the calls are made, e.g. during graph
// capture): the slot this launch stamps, or null.
long long *launch_timeline_slot() {
  static int calls = 0;
  if (!g_profile_buf || !std::getenv("HOM_GEMM_LAUNCH_TIMELINE")) return nullptr;
  return g_profile_buf + 3800 + 6 * (calls++ % 48);
}

void profile_report(const char *what, int tiles, int grid, int num_kb, cudaStream_t stream) {
  if (std::getenv("HOM_GEMM_TIMELINE")) return;  // stamps are read back by the caller
  long long h[16];
  cudaStreamSynchronize(stream);
  cudaMemcpy(h, g_profile_buf, sizeof(h), cudaMemcpyDeviceToHost);
  fprintf(stderr,
          "[hom] %s tiles %d grid %d kblocks %d | producer total %lld wait-empty %lld | mma total %lld "
          "wait-full %lld wait-acc %lld | epilogue total %lld wait-full %lld | odd-CTA producer total "
          "%lld wait-empty %lld | setup %lld kernel %lld cycles, entry %lld ns, exit-entry %lld ns\n",
          what, tiles, grid, num_kb, h[0], h[1], h[2], h[3], h[4], h[5], h[6], h[8], h[9], h[10], h[11],
          h[12], h[13] - h[12]);
}

// 2-D fp16 tensor [outer, inner] (inner contiguous), 128-byte swizzle, zero fill.
bool make_tensor_map_2d(const void *ptr, uint64_t inner, uint64_t outer, uint32_t box_inner,
                        uint32_t box_outer, CUtensorMap *out) {
  MapKey key{ptr, inner, outer, box_inner, box_outer};
  {
    std::lock_guard<std::mutex> lock(g_map_mutex);
    auto it = g_map_cache.find(key);
    if (it != g_map_cache.end()) {
      *out = it->second;
      return true;
    }
  }
  EncodeFn encode = get_encode_fn();
  if (!encode) {
    set_error(HOM_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
    return false;
  }
  cuuint64_t dims[2] = {inner, outer};
  cuuint64_t strides[1] = {inner * 2};
  cuuint32_t box[2] = {box_inner, box_outer};
  cuuint32_t elem_strides[2] = {1, 1};
  CUresult r = encode(out, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void *>(ptr), dims,
                      strides, box, elem_strides, CU_TENSOR_MAP_INTERLEAVE_NONE,
                      CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                      CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_error(HOM_ERR_CUDA, "cuTensorMapEncodeTiled failed (%d) for [%llu x %llu] box [%u x %u]",
              static_cast<int>(r), static_cast<unsigned long long>(outer),
              static_cast<unsigned long long>(inner), box_outer, box_inner);
    return false;
  }
  std::lock_guard<std::mutex> lock(g_map_mutex);
  if (g_map_cache.size() > 8192) g_map_cache.clear();
  g_map_cache.emplace(key, *out);
  return true;
}

// Row-major fp16 matrix [rows, cols] with cols % 64 == 0, seen as a 3-D tensor
// (64 columns, rows, cols / 64 column groups): one box of (64, box_rows, groups) lands in
// shared memory as `groups` consecutive 128-byte-swizzled [box_rows x 64] sub-tiles, so one
// TMA instruction fetches what would otherwise take one 2-D load per 64-column group.
bool make_tensor_map_grouped(const void *ptr, uint64_t cols, uint64_t rows, uint32_t box_rows,
                             uint32_t groups, CUtensorMap *out) {
  MapKey key{ptr, cols, rows, 64u | 0x80000000u, box_rows | (groups << 16)};
  {
    std::lock_guard<std::mutex> lock(g_map_mutex);
    auto it = g_map_cache.find(key);
    if (it != g_map_cache.end()) {
      *out = it->second;
      return true;
    }
  }
  EncodeFn encode = get_encode_fn();
  if (!encode) {
    set_error(HOM_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
    return false;
  }
  cuuint64_t dims[3] = {64, rows, cols / 64};
  cuuint64_t strides[2] = {cols * 2, 128};
  cuuint32_t box[3] = {64, box_rows, groups};
  cuuint32_t elem_strides[3] = {1, 1, 1};
  CUresult r = encode(out, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, const_cast<void *>(ptr), dims,
                      strides, box, elem_strides, CU_TENSOR_MAP_INTERLEAVE_NONE,
                      CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                      CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_error(HOM_ERR_CUDA, "cuTensorMapEncodeTiled (grouped) failed (%d) for [%llu x %llu]",
              static_cast<int>(r), static_cast<unsigned long long>(rows),
              static_cast<unsigned long long>(cols));
    return false;
  }
  std::lock_guard<std::mutex> lock(g_map_mutex);
  if (g_map_cache.size() > 8192) g_map_cache.clear();
  g_map_cache.emplace(key, *out);
  return true;
}

namespace {

template <int BN, bool B_NK>
bool launch_variant(const Problem &pb, cudaStream_t stream) {
  using Cfg = TileCfg<BN>;
  static bool attr_set[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  auto kernel = gemm_f16_kernel<BN, B_NK>;
  if (dev >= 0 && dev < 64 && !attr_set[dev]) {
    if (!check_cuda(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         Cfg::kSmemBytes),
                    "cudaFuncSetAttribute(gemm)"))
      return false;
    attr_set[dev] = true;
  }
  CUtensorMap tmA, tmB, tmD;
  if (!make_tensor_map_2d(pb.A, pb.K, pb.M, BK, BM, &tmA)) return false;
  if (pb.N % 8 == 0) {
    if (!make_tensor_map_2d(pb.D, pb.N, pb.M, 64, 32, &tmD)) return false;
  } else {
    tmD = tmA;  // never dereferenced: the epilogue stores without TMA when N % 8 != 0
  }
  const bool grouped = !B_NK && pb.N % 64 == 0;
  if (B_NK) {
    if (!make_tensor_map_2d(pb.B, pb.K, pb.N, BK, BN, &tmB)) return false;
  } else if (grouped) {
    if (!make_tensor_map_grouped(pb.B, pb.N, pb.K, BK, BN / 64, &tmB)) return false;
  } else {
    if (!make_tensor_map_2d(pb.B, pb.N, pb.K, 64, BK, &tmB)) return false;
  }
  Params p;
  p.b_grouped = grouped ? 1 : 0;
  p.ep.M = static_cast<int>(pb.M);
  p.ep.N = static_cast<int>(pb.N);
  p.K = static_cast<int>(pb.K);
  p.ep.C = pb.C;
  p.ep.ldc = pb.N;
  p.ep.c_mode = pb.c_mode;
  p.ep.D = pb.D;
  p.ep.ldd = pb.N;
  p.ep.alpha = pb.alpha;
  p.ep.beta = pb.beta;
  p.ep.act = pb.act;
  p.ep.row_scale = pb.row_scale;
  p.ep.row_shift = pb.row_shift;
  p.ep.col_sum = pb.col_sum;
  p.ep.unaligned_n = pb.N % 8 != 0 ? 1 : 0;
  const int m_blocks = static_cast<int>((pb.M + BM - 1) / BM);
  p.n_blocks = static_cast<int>((pb.N + BN - 1) / BN);
  p.num_tiles = m_blocks * p.n_blocks;
  p.num_kb = static_cast<int>((pb.K + BK - 1) / BK);
  p.stages = Cfg::kStages;
  if (const char *env = std::getenv("HOM_GEMM_STAGES")) {  // experiment knob
    const int v = std::atoi(env);
    if (v >= 1 && v < Cfg::kStages) p.stages = v;
  }
  p.status = device_status_word();
  p.prof = profile_buffer();
  p.tl = launch_timeline_slot();
  const int grid = p.num_tiles < sm_count() ? p.num_tiles : sm_count();
  const double flops = 2.0 * pb.M * pb.N * pb.K;
  const double bytes = 2.0 * (static_cast<double>(pb.M) * pb.K + static_cast<double>(pb.K) * pb.N +
                              static_cast<double>(pb.M) * pb.N) +
                       (pb.c_mode == 1 ? 2.0 * pb.M * pb.N : pb.c_mode == 2 ? 2.0 * pb.N : 0.0);
  LaunchScope scope(kOpGemm, flops, bytes);
  if (!check_cuda(launch_pdl(kernel, dim3(grid), dim3(kThreads), Cfg::kSmemBytes, stream, 1, tmA, tmB,
                             tmD, p),
                  "gemm kernel launch"))
    return false;
  if (p.prof) profile_report("gemm 1-CTA", p.num_tiles, grid, p.num_kb, stream);
  return check_cuda(cudaGetLastError(), "gemm kernel launch");
}

// D = LayerNorm(fp16(A.B + R)) over the last dimension: one cluster of pb.N / BN CTAs per 128
// rows (grid = tiles); R in pb.C (c_mode 1) or absent.
template <int BN, bool B_NK>
bool launch_ln_variant(const Problem &pb, float eps, cudaStream_t stream) {
  using Cfg = TileCfg<BN>;
  static bool attr_set[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  auto kernel = gemm_f16_kernel<BN, B_NK, true>;
  if (dev >= 0 && dev < 64 && !attr_set[dev]) {
    if (!check_cuda(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         Cfg::kSmemBytes),
                    "cudaFuncSetAttribute(gemm + layernorm)"))
      return false;
    attr_set[dev] = true;
  }
  CUtensorMap tmA, tmB, tmD;
  if (!make_tensor_map_2d(pb.A, pb.K, pb.M, BK, BM, &tmA)) return false;
  if (!make_tensor_map_2d(pb.D, pb.N, pb.M, 64, 32, &tmD)) return false;
  if (B_NK) {
    if (!make_tensor_map_2d(pb.B, pb.K, pb.N, BK, BN, &tmB)) return false;
  } else {
    if (!make_tensor_map_grouped(pb.B, pb.N, pb.K, BK, BN / 64, &tmB)) return false;
  }
  Params p;
  p.b_grouped = B_NK ? 0 : 1;
  p.ep.M = static_cast<int>(pb.M);
  p.ep.N = static_cast<int>(pb.N);
  p.K = static_cast<int>(pb.K);
  p.ep.C = pb.C;
  p.ep.ldc = pb.N;
  p.ep.c_mode = pb.c_mode;
  p.ep.D = pb.D;
  p.ep.ldd = pb.N;
  p.ep.alpha = 1.f;
  p.ep.beta = 1.f;
  p.ep.act = 0;
  p.ep.row_scale = nullptr;
  p.ep.row_shift = nullptr;
  p.ep.col_sum = nullptr;
  p.ep.unaligned_n = 0;
  const int m_blocks = static_cast<int>((pb.M + BM - 1) / BM);
  p.n_blocks = static_cast<int>(pb.N / BN);
  p.num_tiles = m_blocks * p.n_blocks;
  p.num_kb = static_cast<int>((pb.K + BK - 1) / BK);
  p.stages = Cfg::kStages;
  p.status = device_status_word();
  p.prof = nullptr;
  p.tl = nullptr;
  p.ln_eps = eps;
  p.ln_inv_n = 1.f / static_cast<float>(pb.N);
  p.ln_cluster = p.n_blocks;
  const double flops = 2.0 * pb.M * pb.N * pb.K;
  const double bytes = 2.0 * (static_cast<double>(pb.M) * pb.K + static_cast<double>(pb.K) * pb.N +
                              static_cast<double>(pb.M) * pb.N) +
                       (pb.c_mode == 1 ? 2.0 * pb.M * pb.N : 0.0);
  LaunchScope scope(kOpGemm, flops, bytes);
  return check_cuda(launch_pdl(kernel, dim3(p.num_tiles), dim3(kThreads), Cfg::kSmemBytes, stream,
                               static_cast<unsigned>(p.n_blocks), tmA, tmB, tmD, p),
                    "gemm + layernorm kernel launch");
}

struct ShapeRow {
  int64_t m, n, k;
  int act;
  int row;
};

// Tile-table rows: 1-4 = one CTA per 128 x {64,128,192,256} tile; 5, 6 = one CTA pair per
// 256 x {128,256} tile.
struct TileRow {
  int tile_m, tile_n, stages;
  bool pair;
};
const TileRow kTileRows[7] = {
    {0, 0, 0, false},      {128, 64, 6, false},  {128, 128, 5, false}, {128, 192, 4, false},
    {128, 256, 3, false},  {256, 128, 6, true},  {256, 256, 5, true},
};
constexpr int kNumTileRows = 6;

// Per-shape choices for the BERT-base encoder GEMMs (M = batch*seq rows), replacing the
// reference's autotune cache keyed on (M, N, K, activation).
const ShapeRow kShapeTable[] = {
    {4096, 2304, 768, 0, 6},   // base QKV
    {4096, 768, 768, 0, 3},    // base attention output projection (+ residual)
    {4096, 3072, 768, 1, 6},   // base FFN1 + GELU
    {4096, 768, 3072, 0, 3},   // base FFN2 (+ residual)
    {512, 3072, 768, 1, 2},    // single fused GEMM + bias + GELU case
};

}  // namespace

namespace {

// cuTensorMapEncodeTiled without the cache (no host allocation either).
bool encode_map_uncached(const void *ptr, int rank, const cuuint64_t *dims, const cuuint64_t *strides,
                         const cuuint32_t *box, CUtensorMap *out) {
  EncodeFn encode = get_encode_fn();
  if (!encode) {
    set_error(HOM_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
    return false;
  }
  cuuint32_t elem_strides[3] = {1, 1, 1};
  const CUresult r = encode(out, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, static_cast<cuuint32_t>(rank),
                            const_cast<void *>(ptr), dims, strides, box, elem_strides,
                            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                            CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_error(HOM_ERR_CUDA, "cuTensorMapEncodeTiled failed (%d)", static_cast<int>(r));
    return false;
  }
  return true;
}

}  // namespace

// Launches the 128 x 128 single-CTA kernel for `pb` (B as [K, N]) without allocating anything:
// tensor maps are encoded on the stack instead of being cached, the device status word is used
// only if an earlier call already created it, and the SM count comes straight from the
// device attribute.
bool run_fixed_no_alloc(const Problem &pb, cudaStream_t stream) {
  constexpr int BN = 128;
  using Cfg = TileCfg<BN>;
  if (pb.M == 0 || pb.N == 0) return true;
  auto kernel = gemm_f16_kernel<BN, false>;
  if (!check_cuda(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       Cfg::kSmemBytes),
                  "cudaFuncSetAttribute(gemm)"))
    return false;
  int dev = 0, sms = 0;
  cudaGetDevice(&dev);
  if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0)
    sms = 148;
  CUtensorMap tmA, tmB, tmD;
  const bool grouped = pb.N % 64 == 0;
  {
    const cuuint64_t dims[2] = {static_cast<cuuint64_t>(pb.K), static_cast<cuuint64_t>(pb.M)};
    const cuuint64_t strides[1] = {static_cast<cuuint64_t>(pb.K) * 2};
    const cuuint32_t box[2] = {BK, BM};
    if (!encode_map_uncached(pb.A, 2, dims, strides, box, &tmA)) return false;
  }
  if (grouped) {
    const cuuint64_t dims[3] = {64, static_cast<cuuint64_t>(pb.K), static_cast<cuuint64_t>(pb.N / 64)};
    const cuuint64_t strides[2] = {static_cast<cuuint64_t>(pb.N) * 2, 128};
    const cuuint32_t box[3] = {64, BK, BN / 64};
    if (!encode_map_uncached(pb.B, 3, dims, strides, box, &tmB)) return false;
  } else {
    const cuuint64_t dims[2] = {static_cast<cuuint64_t>(pb.N), static_cast<cuuint64_t>(pb.K)};
    const cuuint64_t strides[1] = {static_cast<cuuint64_t>(pb.N) * 2};
    const cuuint32_t box[2] = {64, BK};
    if (!encode_map_uncached(pb.B, 2, dims, strides, box, &tmB)) return false;
  }
  {
    const cuuint64_t dims[2] = {static_cast<cuuint64_t>(pb.N), static_cast<cuuint64_t>(pb.M)};
    const cuuint64_t strides[1] = {static_cast<cuuint64_t>(pb.N) * 2};
    const cuuint32_t box[2] = {64, 32};
    if (!encode_map_uncached(pb.D, 2, dims, strides, box, &tmD)) return false;
  }
  Params p;
  p.ep.M = static_cast<int>(pb.M);
  p.ep.N = static_cast<int>(pb.N);
  p.K = static_cast<int>(pb.K);
  p.ep.C = pb.C;
  p.ep.ldc = pb.N;
  p.ep.c_mode = pb.c_mode;
  p.ep.D = pb.D;
  p.ep.ldd = pb.N;
  p.ep.alpha = pb.alpha;
  p.ep.beta = pb.beta;
  p.ep.act = pb.act;
  p.ep.row_scale = pb.row_scale;
  p.ep.row_shift = pb.row_shift;
  p.ep.col_sum = pb.col_sum;
  p.ep.unaligned_n = pb.N % 8 != 0 ? 1 : 0;
  p.b_grouped = grouped ? 1 : 0;
  const int m_blocks = static_cast<int>((pb.M + BM - 1) / BM);
  p.n_blocks = static_cast<int>((pb.N + BN - 1) / BN);
  p.num_tiles = m_blocks * p.n_blocks;
  p.num_kb = static_cast<int>((pb.K + BK - 1) / BK);
  p.stages = Cfg::kStages;
  p.status = device_status_word_if_ready();
  p.prof = nullptr;
  p.tl = nullptr;
  const int grid = p.num_tiles < sms ? p.num_tiles : sms;
  const double flops = 2.0 * pb.M * pb.N * pb.K;
  const double bytes = 2.0 * (static_cast<double>(pb.M) * pb.K + static_cast<double>(pb.K) * pb.N +
                              static_cast<double>(pb.M) * pb.N);
  LaunchScope scope(kOpGemm, flops, bytes);
  return check_cuda(launch_pdl(kernel, dim3(grid), dim3(kThreads), Cfg::kSmemBytes, stream, 1, tmA, tmB,
                               tmD, p),
                    "gemm kernel launch");
}

// ---- tuned shapes: (M, N, K, activation) -> tile-table row, filled by tune() or a cache file.
// Takes the place of the reference's GemmProfiler timing cache
// (include/NVGPUKernels/GemmProfiler.h:39-41).
namespace {
using TuneKey = std::tuple<int64_t, int64_t, int64_t, int>;
std::map<TuneKey, int> g_tuned;
std::mutex g_tuned_mutex;

void load_env_cache_once() {
  static std::once_flag once;
  std::call_once(once, [] {
    if (const char *path = std::getenv("HOM_TUNE_CACHE")) tune_cache_load(path);
  });
}

__global__ void fill_pattern_kernel(__half *p, size_t n, uint32_t seed, float scale) {
  for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<size_t>(gridDim.x) * blockDim.x) {
    uint32_t h = static_cast<uint32_t>(i) * 2654435761u + seed;
    h ^= h >> 15;
    h *= 2246822519u;
    h ^= h >> 13;
    p[i] = __float2half((static_cast<float>(h & 0xffff) / 32768.f - 1.f) * scale);
  }
}
}  // namespace

int tuned_row(int64_t m, int64_t n, int64_t k, int act) {
  load_env_cache_once();
  std::lock_guard<std::mutex> lock(g_tuned_mutex);
  auto it = g_tuned.find(TuneKey{m, n, k, act});
  return it == g_tuned.end() ? 0 : it->second;
}

int tune_cache_load(const char *path) {
  FILE *f = path ? std::fopen(path, "r") : nullptr;
  if (!f) return -1;
  long long m, n, k;
  int act, row, count = 0;
  std::lock_guard<std::mutex> lock(g_tuned_mutex);
  while (std::fscanf(f, "%lld %lld %lld %d %d", &m, &n, &k, &act, &row) == 5) {
    if (row >= 1 && row <= kNumTileRows) {
      g_tuned[TuneKey{m, n, k, act}] = row;
      ++count;
    }
  }
  std::fclose(f);
  return count;
}

int tune_cache_save(const char *path) {
  FILE *f = path ? std::fopen(path, "w") : nullptr;
  if (!f) return -1;
  std::lock_guard<std::mutex> lock(g_tuned_mutex);
  for (const auto &kv : g_tuned)
    std::fprintf(f, "%lld %lld %lld %d %d\n", static_cast<long long>(std::get<0>(kv.first)),
                 static_cast<long long>(std::get<1>(kv.first)),
                 static_cast<long long>(std::get<2>(kv.first)), std::get<3>(kv.first), kv.second);
  std::fclose(f);
  return static_cast<int>(g_tuned.size());
}

// Times every row of the tile table on scratch buffers of the given shape (the contract of
// GemmProfiler::profile, lib/NVGPUKernels/GemmProfiler.cu:143-236: warm up, then batches of
// launches between two events on one stream; beta != 0 reads C = D like the reference does).
bool tune(int64_t m, int64_t n, int64_t k, int act, float alpha, float beta, bool b_is_nk, int iters,
          int *best_row, float *best_us, float *row_us, cudaStream_t stream) {
  if (m <= 0 || n <= 0 || k <= 0 || k % 8 != 0 || (!b_is_nk && n % 8 != 0)) {
    set_error(HOM_ERR_UNSUPPORTED, "homGemmTune: shape %lld x %lld x %lld is not supported",
              static_cast<long long>(m), static_cast<long long>(n), static_cast<long long>(k));
    return false;
  }
  if (iters < 1) iters = 20;
  __half *a = nullptr, *b = nullptr, *d = nullptr;
  cudaEvent_t e0 = nullptr, e1 = nullptr;
  auto cleanup = [&]() {
    cudaFree(a);
    cudaFree(b);
    cudaFree(d);
    if (e0) cudaEventDestroy(e0);
    if (e1) cudaEventDestroy(e1);
  };
  if (cudaMalloc(&a, sizeof(__half) * m * k) != cudaSuccess || cudaMalloc(&b, sizeof(__half) * k * n) != cudaSuccess ||
      cudaMalloc(&d, sizeof(__half) * m * n) != cudaSuccess || cudaEventCreate(&e0) != cudaSuccess ||
      cudaEventCreate(&e1) != cudaSuccess) {
    cleanup();
    check_cuda(cudaGetLastError(), "homGemmTune allocation");
    set_error(HOM_ERR_CUDA, "homGemmTune: could not allocate the scratch operands");
    return false;
  }
  fill_pattern_kernel<<<592, 256, 0, stream>>>(a, static_cast<size_t>(m) * k, 1u, 1.f);
  fill_pattern_kernel<<<592, 256, 0, stream>>>(b, static_cast<size_t>(k) * n, 2u, 0.03f);
  fill_pattern_kernel<<<592, 256, 0, stream>>>(d, static_cast<size_t>(m) * n, 3u, 0.5f);
  Problem pb;
  pb.M = m;
  pb.N = n;
  pb.K = k;
  pb.A = a;
  pb.B = b;
  pb.b_is_nk = b_is_nk;
  pb.C = beta != 0.f ? d : nullptr;
  pb.c_mode = beta != 0.f ? 1 : 0;
  pb.D = d;
  pb.alpha = alpha;
  pb.beta = beta;
  pb.act = act;
  int best = 0;
  float best_ms = 1e30f;
  bool ok = true;
  for (int row = 1; row <= kNumTileRows && ok; ++row) {
    for (int i = 0; i < 3 && ok; ++i) ok = run(pb, row, stream);
    if (!ok) break;
    cudaEventRecord(e0, stream);
    for (int i = 0; i < iters && ok; ++i) ok = run(pb, row, stream);
    cudaEventRecord(e1, stream);
    if (cudaEventSynchronize(e1) != cudaSuccess) ok = false;
    float ms = 0.f;
    if (ok) cudaEventElapsedTime(&ms, e0, e1);
    const float us = 1e3f * ms / iters;
    if (row_us) row_us[row - 1] = us;
    if (ok && ms < best_ms) {
      best_ms = ms;
      best = row;
    }
  }
  cleanup();
  if (!ok || best == 0) return false;
  {
    std::lock_guard<std::mutex> lock(g_tuned_mutex);
    g_tuned[TuneKey{m, n, k, act}] = best;
  }
  if (best_row) *best_row = best;
  if (best_us) *best_us = 1e3f * best_ms / iters;
  return true;
}

int select_tile_row(int64_t m, int64_t n, int64_t k, int act) {
  if (const char *env = std::getenv("HOM_GEMM_TILE")) {  // experiment knob
    const int v = std::atoi(env);
    if (v >= 1 && v <= kNumTileRows) return v;
  }
  if (const int row = tuned_row(m, n, k, act)) return row;
  for (const ShapeRow &r : kShapeTable)
    if (r.m == m && r.n == n && r.k == k && r.act == act) return r.row;
  // Estimated time = waves x per-tile time.  A wave is 148 single-CTA tiles or 74 pair
  // tiles; the per-tile time grows with the tile's N (MMA columns per K step) plus a fixed
  // part, and a single CTA sustains a lower MMA rate than a pair (its TMA ring is shallower
  // relative to the bytes it has to pull per K step).
  const int sms = sm_count();
  int best = 1;
  double best_cost = 1e300;
  for (int row = 1; row <= kNumTileRows; ++row) {
    const TileRow &t = kTileRows[row];
    const int64_t tiles = ((m + t.tile_m - 1) / t.tile_m) * ((n + t.tile_n - 1) / t.tile_n);
    const int64_t slots = t.pair ? sms / 2 : sms;
    const int64_t waves = (tiles + slots - 1) / slots;
    const double per_tile = t.pair ? t.tile_n + 48.0 : 1.5 * t.tile_n + 48.0;
    const double cost = static_cast<double>(waves) * per_tile;
    if (cost < best_cost - 1e-9) {
      best_cost = cost;
      best = row;
    }
  }
  return best;
}

int query_tile(int64_t m, int64_t n, int64_t k, int act, int *bn, int *stages, int *split_k) {
  const int row = select_tile_row(m, n, k, act);
  if (bn) *bn = kTileRows[row].tile_n;
  if (stages) *stages = kTileRows[row].stages;
  if (split_k) *split_k = 1;
  return row;
}

bool layernorm_fusion_shape(int64_t n, int *cluster_n, int *bn) {
  for (int c : {1, 2, 4, 8}) {
    if (n % c != 0) continue;
    const int64_t w = n / c;
    if (w == 64 || w == 128 || w == 192 || w == 256) {
      if (cluster_n) *cluster_n = c;
      if (bn) *bn = static_cast<int>(w);
      return true;
    }
  }
  return false;
}

bool run_layernorm_fused(const Problem &pb, float eps, cudaStream_t stream) {
  if (pb.M == 0 || pb.N == 0) return true;
  int cluster_n = 0, bn = 0;
  if (!layernorm_fusion_shape(pb.N, &cluster_n, &bn)) {
    set_error(HOM_ERR_UNSUPPORTED,
              "fused GEMM + LayerNorm needs N = c x {64,128,192,256} with c in {1,2,4,8} (got N = %lld)",
              static_cast<long long>(pb.N));
    return false;
  }
  if (pb.b_is_nk) {
    switch (bn) {
      case 64: return launch_ln_variant<64, true>(pb, eps, stream);
      case 128: return launch_ln_variant<128, true>(pb, eps, stream);
      case 192: return launch_ln_variant<192, true>(pb, eps, stream);
      default: return launch_ln_variant<256, true>(pb, eps, stream);
    }
  }
  switch (bn) {
    case 64: return launch_ln_variant<64, false>(pb, eps, stream);
    case 128: return launch_ln_variant<128, false>(pb, eps, stream);
    case 192: return launch_ln_variant<192, false>(pb, eps, stream);
    default: return launch_ln_variant<256, false>(pb, eps, stream);
  }
}

bool run(const Problem &pb, int tile_row, cudaStream_t stream) {
  if (pb.M == 0 || pb.N == 0) return true;
  if (tile_row < 1 || tile_row > kNumTileRows) tile_row = select_tile_row(pb.M, pb.N, pb.K, pb.act);
  const TileRow &t = kTileRows[tile_row];
  if (t.pair) return run_pair(pb, t.tile_n, stream);
  if (pb.b_is_nk) {
    switch (t.tile_n) {
      case 64: return launch_variant<64, true>(pb, stream);
      case 128: return launch_variant<128, true>(pb, stream);
      case 192: return launch_variant<192, true>(pb, stream);
      default: return launch_variant<256, true>(pb, stream);
    }
  }
  switch (t.tile_n) {
    case 64: return launch_variant<64, false>(pb, stream);
    case 128: return launch_variant<128, false>(pb, stream);
    case 192: return launch_variant<192, false>(pb, stream);
    default: return launch_variant<256, false>(pb, stream);
  }
}

}  // namespace gemm
}  // namespace hom
