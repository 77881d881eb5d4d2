// fp16 GEMM on CTA pairs (tcgen05 cta_group::2): a cluster of two CTAs on neighbouring SMs
// computes a 256 x BN2 output tile.  Each CTA loads its own 128 rows of A and its own BN2/2
// columns of B per K block (plain per-CTA TMA loads whose byte counts complete on the even
// CTA's mbarrier), one thread of the even CTA issues tcgen05.mma for the whole 256 x BN2 x 16
// step, and each CTA drains its 128 accumulator rows from its own tensor memory.  Compared
// with one CTA per 128 x 256 tile this halves the B bytes every SM pulls through L2 and
// shared memory for the same MMA time, which is what the TMA ring needs to keep the tensor
// pipe fed; the freed shared memory holds five stages and the epilogue staging.
//
//   warp 0      TMA producer
//   warp 1      tensor-memory allocation (both CTAs) and MMA issue (even CTA only)
//   warps 2-17  epilogue: four warps per tensor-memory lane quarter, each draining one
//               64-column group of the tile: tcgen05.ld, fp32 alpha/beta/bias/erf-GELU, fp16
//               results staged in swizzled shared memory and written out by TMA stores
//
// Hand-offs: full[s] lives in the even CTA (armed by its producer for the bytes of both CTAs);
// empty[s] and acc_full[a] exist in both CTAs and are signalled by tcgen05.commit addressed to
// both; acc_empty[a] lives in the even CTA (32 arrivals: 16 epilogue warps x 2 CTAs).
// A work unit is a 256 x BN2 tile or one of the `split_k` K ranges of a tile (SplitK,
// gemm_epilogue.cuh).
#include <cstdio>
#include <cstdlib>

#include "gemm_epilogue.cuh"
#include "gemm_sm100.cuh"
#include "ptx_sm100.cuh"

namespace hom {
namespace gemm {

using namespace hom::ptx;

namespace {

constexpr int BK = 64;
constexpr int kPairThreads = 32 * (kControlWarps + kEpilogueWarps);
constexpr uint32_t kABytes = 128 * BK * 2;

template <int BN2>
struct PairCfg {
  static constexpr int kHalfN = BN2 / 2;
  static constexpr uint32_t kBBytes = kHalfN * BK * 2;
  static constexpr uint32_t kStageBytes = kABytes + kBBytes;
  static constexpr int kStages = BN2 == 256 ? 5 : 6;
  static constexpr uint32_t kTmemCols = 2 * BN2;  // two accumulators; 512 or 256
  static constexpr uint32_t kStagingBytes = kEpilogueStagingBytes;
  static constexpr uint32_t kBarrierBytes = 8 * (2 * kStages + 4) + 16;
  static constexpr uint32_t kSmemBytes = kStages * kStageBytes + kStagingBytes + kBarrierBytes + 1024;
};

struct PairParams {
  EpilogueParams ep;
  int K;
  int n_blocks, num_tiles, num_kb;
  int stages;
  int b_grouped;  // B [K,N] is fetched through the grouped 3-D tensor map (N % 64 == 0)
  int b_early;    // B is a declared constant: request its first tiles before griddepcontrol.wait
  // Split-K: every tile is cut into `split_k` work units (K-block ranges); num_units = num_tiles
  // * split_k.  Workspace: per (tile, CTA of the pair, epilogue warp) `split_k` fp32 slots and a
  // pair of counters (see SplitK in gemm_epilogue.cuh).
  int split_k, num_units;
  float *ws_slots;
  int *ws_counters;
  int *status;
  HOM_DIAG(long long *prof;)  // optional per-role cycle counters of CTA 0, else null
  HOM_DIAG(long long *tl;)    // optional launch-timeline slot, else null
};

template <int BN2, bool B_NK, bool SPLIT = false, int FORMS = 0, int EPI = 0>
__global__ void __launch_bounds__(kPairThreads, 1)
gemm_f16_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                     const __grid_constant__ CUtensorMap tmD, const PairParams p) {
  using Cfg = PairCfg<BN2>;
  constexpr int STAGES = Cfg::kStages;
  constexpr int HALF = Cfg::kHalfN;
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
  const uint32_t rank = cluster_ctarank();  // 0: even CTA (issues the MMAs), 1: odd CTA
  const int pair = blockIdx.x >> 1;
  const int num_pairs = gridDim.x >> 1;

  HOM_DIAG(unsigned long long g_entry = 0; if (p.tl) asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(g_entry));
           if (p.tl && threadIdx.x == 0) timeline_stamp(p.tl, 0);)
  // The first TMA instruction stalls until its descriptor has been fetched: start those
  // fetches before anything else so that they overlap the barrier and tensor-memory set-up.
  if (threadIdx.x == 64) {
    prefetch_tensormap(&tmB);
    prefetch_tensormap(&tmA);
    prefetch_tensormap(&tmD);
  }
  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(tfull_bar(a), 1);
      mbar_init(tempty_bar(a), 2 * kEpilogueWarps);
    }
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc_pair(smem_u32(const_cast<uint32_t *>(tmem_slot)), Cfg::kTmemCols);
    tmem_relinquish_pair();
  }
  tc_fence_before_sync();
  cluster_sync_all();  // barriers of both CTAs are initialised before anyone signals them
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  // Dependents may be scheduled only now that this grid's CTAs hold their tensor memory.
  pdl_launch_dependents();
  // longest set-up (entry -> barriers, tensor memory and cluster barrier done) over the CTAs, ns
  HOM_DIAG(if (p.tl && threadIdx.x == 0) {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    atomicMax(p.tl + 480, static_cast<long long>(t - g_entry));
  })

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    // Run by the whole warp (coordinates and addresses stay warp-uniform); one elected lane
    // arms the barriers and issues the copies.
    {
      const bool leader = elect_one();
      int s = 0;
      uint32_t ph = 0;
      bool ok = true;
      HOM_DIAG(long long t_wait = 0; const long long t_begin = clock64();)
      const uint32_t full_even_base = map_to_cta(full_bar(0), 0);
      auto full_even = [&](int slot) { return full_even_base + 8u * slot; };
      auto arm = [&](int slot) {
        // The even CTA's producer arms the barrier for the bytes of both CTAs; the odd CTA's
        // copies only count their bytes on it.
        if (rank == 0 && leader) mbar_arrive_expect_tx(full_bar(slot), 2 * Cfg::kStageBytes);
      };
      auto load_b = [&](int slot, int kb, int nb0) {
        const uint32_t b_dst = smem_base + slot * Cfg::kStageBytes + kABytes;
        if (!leader) return;
        if (B_NK) {
          tma_load_2d_pair(b_dst, &tmB, full_even(slot), kb * BK, nb0);
        } else if (p.b_grouped) {
          tma_load_3d_pair(b_dst, &tmB, full_even(slot), 0, kb * BK, nb0 / 64);
        } else {
#pragma unroll
          for (int g = 0; g < HALF / 64; ++g)
            tma_load_2d_pair(b_dst + g * (BK * 128), &tmB, full_even(slot), nb0 + g * 64, kb * BK);
        }
      };
      // When B is a declared constant (weights, which no kernel of the stream writes) the
      // first ring of B tiles is requested before waiting for the previous kernel; A, and a B
      // of unknown origin, only after.
      int pre = 0;
      if (p.b_early && pair < p.num_units) {
        const int tile0 = pair / p.split_k, part0 = pair % p.split_k;
        const int nb0 = (tile0 % p.n_blocks) * BN2 + static_cast<int>(rank) * HALF;
        const int kb0 = part0 * p.num_kb / p.split_k, kb1 = (part0 + 1) * p.num_kb / p.split_k;
        pre = kb1 - kb0 < stages_used ? kb1 - kb0 : stages_used;
        for (int i = 0; i < pre; ++i) {
          arm(i);
          load_b(i, kb0 + i, nb0);
        }
      }
      // longest entry -> first weight tiles requested (just before the dependency wait), ns
      HOM_DIAG(if (p.tl && leader) {
        unsigned long long t;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
        atomicMax(p.tl + 481, static_cast<long long>(t - g_entry));
      })
      pdl_wait();
      HOM_DIAG(if (p.tl && leader) timeline_stamp(p.tl, 2);)
      for (int unit = pair; unit < p.num_units && ok; unit += num_pairs) {
        const int tile = unit / p.split_k, part = unit % p.split_k;
        const int m0 = (tile / p.n_blocks) * 256 + static_cast<int>(rank) * 128;
        const int nb0 = (tile % p.n_blocks) * BN2 + static_cast<int>(rank) * HALF;
        const int kb_begin = part * p.num_kb / p.split_k, kb_end = (part + 1) * p.num_kb / p.split_k;
        for (int kb = kb_begin; kb < kb_end; ++kb) {
          const bool b_done = unit == pair && kb - kb_begin < pre;
          if (!b_done) {
            HOM_DIAG(const long long tw = p.prof ? clock64() : 0;)
            ok = __all_sync(0xffffffffu, mbar_wait(empty_bar(s), ph ^ 1u, abort_flag, p.status,
                                                   kDevWaitTimeoutProducer));
            if (!ok) break;
            HOM_DIAG(if (p.prof) t_wait += clock64() - tw;)
            arm(s);
            load_b(s, kb, nb0);
          }
          if (leader) tma_load_2d_pair(smem_base + s * Cfg::kStageBytes, &tmA, full_even(s), kb * BK, m0);
          if (++s == stages_used) {
            s = 0;
            ph ^= 1u;
          }
        }
      }
      HOM_DIAG(if (p.prof && blockIdx.x < 2 && lane == 0) {
        p.prof[0 + 8 * blockIdx.x] = clock64() - t_begin;
        p.prof[1 + 8 * blockIdx.x] = t_wait;
      })
      if (!ok) {
        // Give copies already in flight time to land before shared memory is released.
        const long long t0 = clock64();
        while (clock64() - t0 < 4000000LL) {
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------- MMA issuer (even CTA only)
    // The whole warp runs the loop so that stage addresses and descriptors stay warp-uniform;
    // one elected lane issues the MMAs and the commits.
    if (rank == 0) {
      constexpr uint32_t idesc = make_idesc_f16(256, BN2, false, !B_NK);
      const bool leader = elect_one();
      int s = 0;
      uint32_t ph = 0;
      bool ok = true;
      int it = 0;
      HOM_DIAG(long long t_full = 0, t_acc = 0; const long long t_begin = clock64();)
      for (int unit = pair; unit < p.num_units && ok; unit += num_pairs, ++it) {
        const int part = unit % p.split_k;
        const int num_kb = (part + 1) * p.num_kb / p.split_k - part * p.num_kb / p.split_k;
        const int acc = it & 1;
        const uint32_t acc_ph = (it >> 1) & 1;
        HOM_DIAG(const long long ta = p.prof ? clock64() : 0;)
        ok = __all_sync(0xffffffffu,
                        mbar_wait(tempty_bar(acc), acc_ph ^ 1u, abort_flag, p.status, kDevWaitTimeoutMma));
        if (!ok) break;
        HOM_DIAG(if (p.prof) t_acc += clock64() - ta;)
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + acc * BN2;
        bool have = false;  // full[s] already seen complete by the probe of the previous block
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!have) {
            HOM_DIAG(const long long tw = p.prof ? clock64() : 0;)
            ok = __all_sync(0xffffffffu,
                            mbar_wait(full_bar(s), ph, abort_flag, p.status, kDevWaitTimeoutMma));
            if (!ok) break;
            HOM_DIAG(if (p.prof) t_full += clock64() - tw;)
          }
          have = false;
          tc_fence_after_sync();
          HOM_DIAG(if (p.tl && it == 0 && kb == 0 && leader) timeline_stamp(p.tl, 6);)
          const uint32_t a_addr = smem_base + s * Cfg::kStageBytes;
          const uint32_t b_addr = a_addr + kABytes;
          const int s_next = s + 1 == stages_used ? 0 : s + 1;
          const uint32_t ph_next = s_next == 0 ? ph ^ 1u : ph;
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) {
            const uint64_t da = make_smem_desc_sw128(a_addr + k * 32, 16, 1024);
            const uint64_t db = B_NK ? make_smem_desc_sw128(b_addr + k * 32, 16, 1024)
                                     : make_smem_desc_sw128(b_addr + k * 2048, BK * 128, 1024);
            if (leader) tc_mma_f16_ss_pair(d_tmem, da, db, idesc, (kb | k) != 0 ? 1u : 0u);
            // Probe the next stage while the tensor pipe is busy with what was just queued.
            if (k == 1 && kb + 1 < num_kb)
              have = __all_sync(0xffffffffu, mbar_test_wait(full_bar(s_next), ph_next));
          }
          if (leader) tc_commit_pair(empty_bar(s), 0x3);  // frees the stage in both CTAs
          s = s_next;
          ph = ph_next;
        }
        if (ok && leader) tc_commit_pair(tfull_bar(acc), 0x3);  // accumulator ready in both CTAs
      }
      HOM_DIAG(if (p.prof && blockIdx.x == 0 && lane == 0) {
        p.prof[2] = clock64() - t_begin;
        p.prof[3] = t_full;
        p.prof[4] = t_acc;
      })
    }
  } else if (warp >= kControlWarps) {
    // --------------------------------------------------------------- epilogue
    const int quarter = warp & 3;       // tensor-memory lanes [32*quarter, +32)
    const int group = (warp - kControlWarps) >> 2;  // which 64-column group of the tile
    const int col_begin = group * 64;
    const bool active = col_begin < BN2;
    const uint32_t stage_smem = staging_base + (warp - kControlWarps) * kEpilogueStageBytes;
    int it = 0;
    HOM_DIAG(long long t_wait = 0; const long long t_begin = clock64();)
    pdl_wait();  // C may be produced, and D still read, by the previous kernel
    float2 next_col_sums = make_float2(0.f, 0.f);
    if constexpr ((FORMS & kFormLnA) != 0) {
      if (active && pair < p.num_units)
        next_col_sums = epilogue_load_col_sums(p.ep, (pair % p.n_blocks) * BN2 + col_begin, lane);
    }
    for (int unit = pair; unit < p.num_units; unit += num_pairs, ++it) {
      const int tile = unit / p.split_k;
      const int acc = it & 1;
      const uint32_t acc_ph = (it >> 1) & 1;
      const int m0 = (tile / p.n_blocks) * 256 + static_cast<int>(rank) * 128;
      const int n0 = (tile % p.n_blocks) * BN2 + col_begin;
      uint4 cval[8];
      SplitK sk;
      if constexpr (SPLIT) {
        // this warp's block of the tile: (tile, CTA of the pair, epilogue warp)
        const size_t block = (static_cast<size_t>(tile) * 2 + rank) * kEpilogueWarps + (warp - kControlWarps);
        sk.parts = p.split_k;
        sk.part = unit % p.split_k;
        sk.slot = p.ws_slots + block * kSplitSlotFloats;
        sk.counter = p.ws_counters + block;
      } else {
        if constexpr (EPI == kEpiGeneric || EPI == kEpiAddC) {
          if (active) epilogue_load_c<0, 8, EPI != kEpiGeneric || FORMS != 0>(p.ep, m0 + quarter * 32 + lane, n0, cval);
        }
      }
      RowAffine ra;
      float2 col_sums = make_float2(0.f, 0.f);
      if constexpr ((FORMS & (kFormLnA | kFormLnR)) != 0) {
        if (active) ra = epilogue_row_affine(p.ep, m0 + quarter * 32 + lane);
      }
      if constexpr ((FORMS & kFormLnA) != 0) {
        col_sums = next_col_sums;
        const int next = unit + num_pairs;
        if (active && next < p.num_units)
          next_col_sums = epilogue_load_col_sums(p.ep, (next % p.n_blocks) * BN2 + col_begin, lane);
      }
      HOM_DIAG(const long long tw = p.prof ? clock64() : 0;)
      bool ok = mbar_wait(tfull_bar(acc), acc_ph, abort_flag, p.status, kDevWaitTimeoutEpilogue);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      HOM_DIAG(if (p.prof) t_wait += clock64() - tw;)
      HOM_DIAG(if (p.tl && warp == kControlWarps && lane == 0 && unit + num_pairs >= p.num_units)
                   timeline_stamp(p.tl, 8);)
      tc_fence_after_sync();
      auto release = [&]() {
        if (lane == 0) {
          if (rank == 0) mbar_arrive(tempty_bar(acc));
          else mbar_arrive_cluster(map_to_cta(tempty_bar(acc), 0));
        }
      };
      const uint32_t t_row =
          tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + acc * BN2 + col_begin;
      if (!epilogue_warp_block<SPLIT, FORMS, EPI>(p.ep, &tmD, t_row, m0 + quarter * 32, n0, active, stage_smem, lane,
                                             cval, release, sk, abort_flag, p.status, ra, col_sums))
        break;
    }
    // A store still in flight reads this warp's staging tile: let it finish reading.
    if (lane == 0) bulk_wait_group_read_0();
    __syncwarp();
    HOM_DIAG(if (p.prof && blockIdx.x == 0 && threadIdx.x == 32 * kControlWarps) {
      p.prof[5] = clock64() - t_begin;
      p.prof[6] = t_wait;
    })
  }

  // Nobody leaves while the other CTA may still read this CTA's shared memory (MMA operand
  // fetch) or signal its barriers.
  tc_fence_before_sync();
  cluster_sync_all();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc_pair(tmem_base, Cfg::kTmemCols);
  }
  HOM_DIAG(if (p.tl && threadIdx.x == 0) timeline_stamp(p.tl, 4);)
}

template <int BN2, bool B_NK>
bool launch_pair_variant(const Problem &pb, int split_k, cudaStream_t stream) {
  using Cfg = PairCfg<BN2>;
  static bool attr_set[64] = {};
  static int max_clusters[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) dev = 0;
  // the whole-K kernel without LayerNorm forms: generic, or one of the three specialised epilogues
  const int epi = epilogue_kind(pb);
  auto kernel = epi == kEpiPlain  ? gemm_f16_pair_kernel<BN2, B_NK, false, 0, kEpiPlain>
                : epi == kEpiGelu ? gemm_f16_pair_kernel<BN2, B_NK, false, 0, kEpiGelu>
                : epi == kEpiAddC ? gemm_f16_pair_kernel<BN2, B_NK, false, 0, kEpiAddC>
                                  : gemm_f16_pair_kernel<BN2, B_NK>;
  auto kernel_split = gemm_f16_pair_kernel<BN2, B_NK, true>;
  // the LayerNorm forms of the epilogue: on A only / on the residual + statistics / any mix
  const int forms = layernorm_forms(pb);
  auto kernel_forms = forms == kFormLnA ? gemm_f16_pair_kernel<BN2, B_NK, false, kFormLnA>
                      : (forms & kFormLnA) == 0 ? gemm_f16_pair_kernel<BN2, B_NK, false, kFormLnR | kFormStats>
                                                : gemm_f16_pair_kernel<BN2, B_NK, false, kFormLnA | kFormLnR | kFormStats>;

  cudaLaunchConfig_t cfg = {};
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = pdl_enabled() ? 1 : 0;
  cfg.attrs = attr;
  cfg.numAttrs = 2;
  cfg.blockDim = dim3(kPairThreads);
  cfg.dynamicSmemBytes = Cfg::kSmemBytes;
  cfg.stream = stream;

  if (!attr_set[dev]) {
    if (!check_cuda(cudaFuncSetAttribute(gemm_f16_pair_kernel<BN2, B_NK>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         Cfg::kSmemBytes),
                    "cudaFuncSetAttribute(gemm pair)") ||
        !check_cuda(cudaFuncSetAttribute(gemm_f16_pair_kernel<BN2, B_NK, false, 0, kEpiPlain>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes),
                    "cudaFuncSetAttribute(gemm pair, plain)") ||
        !check_cuda(cudaFuncSetAttribute(gemm_f16_pair_kernel<BN2, B_NK, false, 0, kEpiGelu>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes),
                    "cudaFuncSetAttribute(gemm pair, GELU)") ||
        !check_cuda(cudaFuncSetAttribute(gemm_f16_pair_kernel<BN2, B_NK, false, 0, kEpiAddC>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes),
                    "cudaFuncSetAttribute(gemm pair, + C)") ||
        !check_cuda(cudaFuncSetAttribute(gemm_f16_pair_kernel<BN2, B_NK, false, kFormLnA>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes),
                    "cudaFuncSetAttribute(gemm pair, LayerNorm on A)") ||
        !check_cuda(cudaFuncSetAttribute(gemm_f16_pair_kernel<BN2, B_NK, false, kFormLnR | kFormStats>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes),
                    "cudaFuncSetAttribute(gemm pair, LayerNorm on the residual)") ||
        !check_cuda(cudaFuncSetAttribute(gemm_f16_pair_kernel<BN2, B_NK, false, kFormLnA | kFormLnR | kFormStats>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes),
                    "cudaFuncSetAttribute(gemm pair, LayerNorm forms)") ||
        !check_cuda(cudaFuncSetAttribute(kernel_split, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         Cfg::kSmemBytes),
                    "cudaFuncSetAttribute(gemm pair, split-K)"))
      return false;
    // How many CTA pairs the device can hold at once (pairs need neighbouring SMs).
    cfg.gridDim = dim3(2 * (sm_count() / 2));
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, kernel, &cfg) != cudaSuccess || n <= 0) {
      cudaGetLastError();
      n = sm_count() / 2;
    }
    HOM_DIAG(if (const char *env = std::getenv("HOM_GEMM_PAIRS")) {  // experiment knob
      const int v = std::atoi(env);
      if (v >= 1) n = v;
    }
    if (std::getenv("HOM_DEBUG"))
      fprintf(stderr, "[hom] gemm pair BN2=%d nk=%d: %d co-resident CTA pairs\n", BN2, int(B_NK), n);)
    max_clusters[dev] = n;
    attr_set[dev] = true;
  }

  CUtensorMap tmA, tmB, tmD;
  if (!make_tensor_map_2d(pb.A, pb.K, pb.M, BK, 128, &tmA)) return false;
  if (pb.N % 8 == 0) {
    if (!make_tensor_map_2d(pb.D, pb.N, pb.M, 64, 32, &tmD)) return false;
  } else {
    tmD = tmA;  // never dereferenced: the epilogue stores without TMA when N % 8 != 0
  }
  const bool grouped = !B_NK && pb.N % 64 == 0;
  if (B_NK) {
    if (!make_tensor_map_2d(pb.B, pb.K, pb.N, BK, Cfg::kHalfN, &tmB)) return false;
  } else if (grouped) {
    if (!make_tensor_map_grouped(pb.B, pb.N, pb.K, BK, Cfg::kHalfN / 64, &tmB)) return false;
  } else {
    if (!make_tensor_map_2d(pb.B, pb.N, pb.K, 64, BK, &tmB, pb.ldb)) return false;
  }
  PairParams p;
  p.b_grouped = grouped ? 1 : 0;
  p.b_early = pb.b_const ? 1 : 0;
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
  p.ep.a_partials = pb.a_partials;
  p.ep.r_partials = pb.r_partials;
  p.ep.a_groups = pb.a_groups;
  p.ep.r_groups = pb.r_groups;
  p.ep.a_inv_n = pb.K > 0 ? 1.f / static_cast<float>(pb.K) : 0.f;
  p.ep.r_inv_n = pb.N > 0 ? 1.f / static_cast<float>(pb.N) : 0.f;
  p.ep.ln_eps = pb.ln_eps;
  p.ep.unaligned_n = pb.N % 8 != 0 ? 1 : 0;
  p.ep.row_partials = pb.row_partials;
  HOM_DIAG(p.ep.dbg = std::getenv("HOM_EPI_DBG") ? std::atoi(std::getenv("HOM_EPI_DBG")) : 0;)
  p.ep.M = static_cast<int>(pb.M);
  p.ep.N = static_cast<int>(pb.N);
  p.K = static_cast<int>(pb.K);
  const int m_blocks = static_cast<int>((pb.M + 255) / 256);
  p.n_blocks = static_cast<int>((pb.N + BN2 - 1) / BN2);
  p.num_tiles = m_blocks * p.n_blocks;
  p.num_kb = static_cast<int>((pb.K + BK - 1) / BK);
  p.stages = Cfg::kStages;
  HOM_DIAG(if (const char *env = std::getenv("HOM_GEMM_STAGES")) {  // experiment knob
    const int v = std::atoi(env);
    if (v >= 1 && v < Cfg::kStages) p.stages = v;
  })
  p.status = device_status_word();
  HOM_DIAG(p.prof = profile_buffer(); p.tl = launch_timeline_slot();)
  p.split_k = split_k < 1 || has_layernorm_form(pb) ? 1 : split_k > 16 ? 16 : split_k;
  if (p.split_k > p.num_kb) p.split_k = p.num_kb;
  p.num_units = p.num_tiles * p.split_k;
  p.ws_slots = nullptr;
  p.ws_counters = nullptr;
  if (p.split_k > 1) {
    const size_t blocks = static_cast<size_t>(p.num_tiles) * 2 * kEpilogueWarps;
    SplitWorkspace ws;
    if (!split_workspace(blocks * kSplitSlotFloats, blocks, stream, &ws)) return false;
    p.ws_slots = ws.slots;
    p.ws_counters = ws.counters;
  }
  const int pairs = p.num_units < max_clusters[dev] ? p.num_units : max_clusters[dev];
  cfg.gridDim = dim3(2 * pairs);
  const double flops = 2.0 * pb.M * pb.N * pb.K;
  const double bytes = 2.0 * (static_cast<double>(pb.M) * pb.K + static_cast<double>(pb.K) * pb.N +
                              static_cast<double>(pb.M) * pb.N) +
                       (pb.c_mode == 1 ? 2.0 * pb.M * pb.N : pb.c_mode == 2 ? 2.0 * pb.N : 0.0);
  LaunchScope scope(kOpGemm, flops, bytes);
  if (!check_cuda(cudaLaunchKernelEx(&cfg, forms != 0 ? kernel_forms : p.split_k > 1 ? kernel_split : kernel,
                                     tmA, tmB, tmD, p),
                  "gemm pair kernel launch"))
    return false;
  HOM_DIAG(if (p.prof) profile_report("gemm CTA-pair", p.num_tiles, 2 * pairs, p.num_kb, stream);)
  return check_cuda(cudaGetLastError(), "gemm pair kernel launch");
}

}  // namespace

bool run_pair(const Problem &pb, int bn2, int split_k, cudaStream_t stream) {
  if (pb.b_is_nk) {
    return bn2 == 128 ? launch_pair_variant<128, true>(pb, split_k, stream)
                      : launch_pair_variant<256, true>(pb, split_k, stream);
  }
  return bn2 == 128 ? launch_pair_variant<128, false>(pb, split_k, stream)
                    : launch_pair_variant<256, false>(pb, split_k, stream);
}

}  // namespace gemm
}  // namespace hom
