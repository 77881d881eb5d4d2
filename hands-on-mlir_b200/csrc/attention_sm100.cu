// Packed-QKV padded bidirectional attention for sm_100a, head_dim 64.
//
// One CTA per (128-query tile, head, batch).  Q, K and V tiles are 128 x 64 fp16 boxes
// that TMA lifts straight out of the packed [bs*seq, 3*heads*64] tensor into
// 128-byte-swizzled shared memory.  S = Q.K^T (128 x 128, fp32) and O_j = P.V (128 x 64)
// are tcgen05.mma results in tensor memory; the softmax runs one query row per thread in
// fp32 with an online rescale across 128-wide KV tiles, so sequence lengths 128 and 512
// share one code path and S / P never touch HBM.  KV tiles beyond a sequence's valid
// length are skipped, the ragged tile is masked, and padded query rows are written as zeros.
//
// Replaces the reference's cuDNN fused attention behind TransformerEngine
// (include/NVGPUKernels/BertAttentionRunner.h:52-136: layout BS3HD, no bias, padding mask,
// no dropout, inference).
#include <cstdio>
#include <cstdlib>
#include <mutex>
#include <unordered_map>

#include "attention_sm100.cuh"
#include "gemm_sm100.cuh"
#include "hom_diag.cuh"
#include "ptx_sm100.cuh"

namespace hom {
namespace attention {

using namespace hom::ptx;

namespace {

constexpr int kTile = 128;   // query rows per CTA and KV rows per step
constexpr int kHeadDim = 64;
constexpr int kThreads = 256;  // two threads per query row
constexpr uint32_t kTileBytes = kTile * kHeadDim * 2;  // 16 KB
constexpr uint32_t kSmemQ = 0;
constexpr uint32_t kSmemK = kTileBytes;
constexpr uint32_t kSmemV = 2 * kTileBytes;
constexpr uint32_t kSmemP = 3 * kTileBytes;  // two 128 x 64 sub-tiles
constexpr uint32_t kSmemBar = 5 * kTileBytes;
constexpr uint32_t kSmemBytes = kSmemBar + 64 + 2 * kTile * 4 + 1024;  // + row max / sum exchange
constexpr uint32_t kTmemCols = 256;  // S: columns [0,128), O: columns [128,192)

struct Params {
  const int *cu_seqlens;  // [bs + 1]
  __half *out;            // [bs*seq, heads*64]
  int seq, heads;
  float scale_log2;  // softmax scale * log2(e)
  int *status;
  HOM_DIAG(long long *prof;)     // phase stamps of two CTAs (HOM_ATTN_PROFILE), else null
  HOM_DIAG(int timeline_slot;)   // >= 0: record first/last CTA entry and exit times instead
};

__device__ __forceinline__ unsigned long long global_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}

__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// Any sequence length: online softmax over 128-key tiles.  A query row is shared by threads
// `row` and `row + 128`: each owns 64 of a tile's 128 key columns (one 128-byte P sub-tile
// row) and 32 of the 64 output columns, whose running sum lives in its registers.
__global__ void __launch_bounds__(kThreads, 2)
attention_f16_kernel(const __grid_constant__ CUtensorMap tmQKV, const Params p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t smem_base = (raw_addr + 1023u) & ~1023u;
  uint8_t *smem_gen = smem_raw + (smem_base - raw_addr);

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int row = tid & (kTile - 1);
  const int hf = tid >> 7;
  const int q_tile = blockIdx.x, head = blockIdx.y, batch = blockIdx.z;
  const int hidden = p.heads * kHeadDim;
  const int q0 = q_tile * kTile;

  pdl_wait();  // cu_seqlens and the packed QKV come from earlier kernels of the stream
  int len = p.cu_seqlens[batch + 1] - p.cu_seqlens[batch];
  len = max(0, min(len, p.seq));

  const int q_idx = q0 + row;
  __half *out_seg = p.out + (static_cast<long long>(batch) * p.seq + q_idx) * hidden + head * kHeadDim + hf * 32;

  if (q0 >= len) {
    // Entirely padded query tile.
    if (q_idx < p.seq) {
      const uint4 z = make_uint4(0, 0, 0, 0);
#pragma unroll
      for (int g = 0; g < 4; ++g) reinterpret_cast<uint4 *>(out_seg)[g] = z;
    }
    return;
  }

  const uint32_t bar_q = smem_base + kSmemBar;
  const uint32_t bar_k = bar_q + 8, bar_v = bar_q + 16, bar_s = bar_q + 24, bar_o = bar_q + 32;
  volatile uint32_t *tmem_slot = reinterpret_cast<volatile uint32_t *>(smem_gen + kSmemBar + 40);
  volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);
  float *xchg = reinterpret_cast<float *>(smem_gen + kSmemBar + 64);  // [2][128] row maxima / sums

  if (tid == 0) {
    mbar_init(bar_q, 1);
    mbar_init(bar_k, 1);
    mbar_init(bar_v, 1);
    mbar_init(bar_s, 1);
    mbar_init(bar_o, 1);
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 0) {
    tmem_alloc(smem_u32(const_cast<uint32_t *>(tmem_slot)), kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  // Dependents may be scheduled only now that this CTA holds its tensor memory (a CTA that
  // returned above counts as having triggered).
  pdl_launch_dependents();
  const uint32_t tmem_s = tmem_base;
  const uint32_t tmem_o = tmem_base + 128;
  const uint32_t lane_sel = static_cast<uint32_t>((warp & 3) * 32) << 16;

  const int n_kv = (len + kTile - 1) / kTile;
  const int row_base = batch * p.seq;
  const int col_q = head * kHeadDim;
  const int col_k = hidden + head * kHeadDim;
  const int col_v = 2 * hidden + head * kHeadDim;

  // Warp 0 runs the copy / MMA issue code as a whole (addresses and descriptors stay
  // warp-uniform); one elected lane executes the asynchronous instructions.
  const bool leader = warp == 0 && elect_one();
  uint32_t armed_k = 0, armed_v = 0;  // counted by every lane of warp 0, used by thread 0
  if (warp == 0) armed_k = armed_v = 1;
  if (leader) {
    prefetch_tensormap(&tmQKV);
    mbar_arrive_expect_tx(bar_q, kTileBytes);
    tma_load_2d(smem_base + kSmemQ, &tmQKV, bar_q, col_q, row_base + q0);
    mbar_arrive_expect_tx(bar_k, kTileBytes);
    tma_load_2d(smem_base + kSmemK, &tmQKV, bar_k, col_k, row_base);
    mbar_arrive_expect_tx(bar_v, kTileBytes);
    tma_load_2d(smem_base + kSmemV, &tmQKV, bar_v, col_v, row_base);
  }

  constexpr uint32_t idesc_s = make_idesc_f16(kTile, kTile, false, false);
  constexpr uint32_t idesc_o = make_idesc_f16(kTile, kHeadDim, false, true);

  const float2 scale2 = make_float2(p.scale_log2, p.scale_log2);
  float m_run = -INFINITY, l_run = 0.f;  // l_run: this thread's half of the row sum
  float2 o_acc[16];                      // output columns [32 * hf, +32)
#pragma unroll
  for (int i = 0; i < 16; ++i) o_acc[i] = make_float2(0.f, 0.f);

  bool ok = true;
  for (int j = 0; j < n_kv && ok; ++j) {
    const uint32_t ph = j & 1;
    // ---- S = Q.K_j^T
    if (warp == 0) {
      bool w = true;
      if (j == 0) w = mbar_wait(bar_q, 0, abort_flag, p.status, kDevWaitTimeoutAttention);
      w = w && mbar_wait(bar_k, ph, abort_flag, p.status, kDevWaitTimeoutAttention);
      if (__all_sync(0xffffffffu, w)) {
        tc_fence_after_sync();
#pragma unroll
        for (int k = 0; k < kHeadDim / 16; ++k) {
          const uint64_t da = make_smem_desc_sw128(smem_base + kSmemQ + k * 32, 16, 1024);
          const uint64_t db = make_smem_desc_sw128(smem_base + kSmemK + k * 32, 16, 1024);
          if (leader) tc_mma_f16_ss(tmem_s, da, db, idesc_s, k != 0 ? 1u : 0u);
        }
        if (leader) tc_commit(bar_s);
      }
    }
    ok = mbar_wait(bar_s, ph, abort_flag, p.status, kDevWaitTimeoutAttention);
    ok = __syncthreads_and(ok);
    if (!ok) break;
    tc_fence_after_sync();
    if (warp == 0 && j + 1 < n_kv) {  // K buffer is free once S has been computed
      if (leader) {
        mbar_arrive_expect_tx(bar_k, kTileBytes);
        tma_load_2d(smem_base + kSmemK, &tmQKV, bar_k, col_k, row_base + (j + 1) * kTile);
      }
      ++armed_k;
    }

    // ---- softmax over this KV tile; columns [0, valid) are real keys
    const int kv0 = j * kTile;
    const int valid = min(kTile, len - kv0);
    float m_part = -INFINITY;
#pragma unroll 1
    for (int c = 2 * hf; c < 2 * hf + 2 && c * 32 < valid; ++c) {
      uint32_t r[32];
      tmem_ld_32x32(tmem_s + lane_sel + c * 32, r);
      tmem_ld_wait();
      if ((c + 1) * 32 <= valid) {
        float m0 = m_part, m1 = -INFINITY;
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          const float2 x = __fmul2_rn(make_float2(__uint_as_float(r[i]), __uint_as_float(r[i + 1])), scale2);
          m0 = fmaxf(m0, x.x);
          m1 = fmaxf(m1, x.y);
        }
        m_part = fmaxf(m0, m1);
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i)
          if (c * 32 + i < valid) m_part = fmaxf(m_part, __uint_as_float(r[i]) * p.scale_log2);
      }
    }
    xchg[hf * kTile + row] = m_part;
    __syncthreads();
    const float m_new = fmaxf(m_run, fmaxf(m_part, xchg[(hf ^ 1) * kTile + row]));
    const float corr = ex2_approx(m_run - m_new);  // 0 on the first tile (m_run = -inf)
    float2 l2 = make_float2(0.f, 0.f);
    {
      const float2 neg_m2 = make_float2(-m_new, -m_new);
      const uint32_t sub = smem_base + kSmemP + hf * kTileBytes + row * 128;
#pragma unroll 1
      for (int c = 2 * hf; c < 2 * hf + 2 && c * 32 < valid; ++c) {
        uint32_t r[32];
        tmem_ld_32x32(tmem_s + lane_sel + c * 32, r);
        tmem_ld_wait();
        const bool full = (c + 1) * 32 <= valid;
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          uint32_t w[4];
#pragma unroll
          for (int jj = 0; jj < 4; ++jj) {
            const int i0 = g * 8 + 2 * jj;
            const float2 x = __ffma2_rn(make_float2(__uint_as_float(r[i0]), __uint_as_float(r[i0 + 1])),
                                        scale2, neg_m2);
            float2 e = make_float2(ex2_approx(x.x), ex2_approx(x.y));
            if (!full) {
              e.x = (c * 32 + i0 < valid) ? e.x : 0.f;
              e.y = (c * 32 + i0 + 1 < valid) ? e.y : 0.f;
            }
            l2 = __fadd2_rn(l2, e);
            const __half2 h = __floats2half2_rn(e.x, e.y);
            w[jj] = *reinterpret_cast<const uint32_t *>(&h);
          }
          const uint32_t chunk = (c & 1) * 4 + g;
          const uint32_t addr = sub + ((chunk ^ (row & 7)) << 4);
          asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(w[0]), "r"(w[1]),
                       "r"(w[2]), "r"(w[3])
                       : "memory");
        }
      }
    }
    l_run = fmaf(l_run, corr, l2.x + l2.y);
    fence_proxy_async_smem();
    tc_fence_before_sync();
    __syncthreads();  // P complete, and every thread is done reading S

    // ---- O_j = P.V_j over the key groups that hold a valid key
    if (warp == 0) {
      if (__all_sync(0xffffffffu, mbar_wait(bar_v, ph, abort_flag, p.status, kDevWaitTimeoutAttention))) {
        tc_fence_after_sync();
        const int k_steps = (valid + 15) >> 4;
        for (int k = 0; k < k_steps; ++k) {
          const uint64_t da = make_smem_desc_sw128(
              smem_base + kSmemP + (k >> 2) * kTileBytes + (k & 3) * 32, 16, 1024);
          // V tile: 128 kv rows of 128 B; N (= d) contiguous, 16 kv rows = 2048 B.
          const uint64_t db = make_smem_desc_sw128(smem_base + kSmemV + k * 2048, kTileBytes, 1024);
          if (leader) tc_mma_f16_ss(tmem_o, da, db, idesc_o, k != 0 ? 1u : 0u);
        }
        if (leader) tc_commit(bar_o);
      }
    }
    ok = mbar_wait(bar_o, ph, abort_flag, p.status, kDevWaitTimeoutAttention);
    ok = __syncthreads_and(ok);
    if (!ok) break;
    tc_fence_after_sync();
    if (warp == 0 && j + 1 < n_kv) {  // V buffer is free once P.V has been computed
      if (leader) {
        mbar_arrive_expect_tx(bar_v, kTileBytes);
        tma_load_2d(smem_base + kSmemV, &tmQKV, bar_v, col_v, row_base + (j + 1) * kTile);
      }
      ++armed_v;
    }
    {
      uint32_t r[32];
      tmem_ld_32x32(tmem_o + lane_sel + hf * 32, r);
      tmem_ld_wait();
      const float2 corr2 = make_float2(corr, corr);
#pragma unroll
      for (int i = 0; i < 16; ++i)
        o_acc[i] = __ffma2_rn(o_acc[i], corr2,
                              make_float2(__uint_as_float(r[2 * i]), __uint_as_float(r[2 * i + 1])));
    }
    m_run = m_new;
  }

  if (ok) {
    xchg[hf * kTile + row] = l_run;
    __syncthreads();
    const float l_row = l_run + xchg[(hf ^ 1) * kTile + row];
    if (q_idx < p.seq) {
      const bool real_row = q_idx < len && l_row > 0.f;
      const float inv = real_row ? 1.f / l_row : 0.f;
      const float2 inv2 = make_float2(inv, inv);
#pragma unroll
      for (int g = 0; g < 4; ++g) {
        uint4 o = make_uint4(0, 0, 0, 0);
        if (real_row) {
          __half2 *o2 = reinterpret_cast<__half2 *>(&o);
#pragma unroll
          for (int jj = 0; jj < 4; ++jj) {
            const float2 v = __fmul2_rn(o_acc[g * 4 + jj], inv2);
            o2[jj] = __floats2half2_rn(v.x, v.y);
          }
        }
        reinterpret_cast<uint4 *>(out_seg)[g] = o;
      }
    }
  } else if (tid == 0) {
    // Let copies that are still in flight land before the shared memory is released.
    const long long t0 = clock64();
    if (armed_k) while (!mbar_try_wait(bar_k, (armed_k - 1) & 1) && clock64() - t0 < 200000000LL) {}
    if (armed_v) while (!mbar_try_wait(bar_v, (armed_v - 1) & 1) && clock64() - t0 < 400000000LL) {}
    while (!mbar_try_wait(bar_q, 0) && clock64() - t0 < 600000000LL) {}
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

// ---------------------------------------------------------------------------------------
// Sequences of at most 128 tokens: one KV tile per (batch, head), so nothing is rescaled.
// P overwrites the Q|K tiles once S has been computed from them, O reuses S's tensor-memory
// columns, and the finished 128 x 64 output tile is staged over the V tile and written by one
// TMA store through a 3-D [hidden, seq, batch] view of the output (rows beyond seq are
// clipped).  48 KB of shared memory and 128 tensor-memory columns per CTA let four CTAs share
// an SM, which is what hides the load -> MMA -> softmax -> MMA -> store latency chain.
constexpr int kThreads1 = 256;  // two threads per query row
constexpr uint32_t kXchgBytes = 2 * 2 * kTile * 4;  // row maxima and row sums of both halves
constexpr uint32_t kSmemBytes1 = 3 * kTileBytes + 64 + kXchgBytes + 1024;

// A query row is shared by threads `row` and `row + 128`: each owns 64 of the 128 key
// columns (one 128-byte P sub-tile row) and 32 of the 64 output columns.  Only the 32-column
// chunks that hold valid keys are read, the chunk that holds the boundary is masked, and the
// P.V product stops at the last 16-key group with a valid key.
__global__ void __launch_bounds__(kThreads1, 4)
attention_f16_single_tile_kernel(const __grid_constant__ CUtensorMap tmQKV,
                                 const __grid_constant__ CUtensorMap tmOut, const Params p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t smem_base = (raw_addr + 1023u) & ~1023u;
  uint8_t *smem_gen = smem_raw + (smem_base - raw_addr);

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int row = tid & (kTile - 1);
  const int hf = tid >> 7;  // which half of the key columns / output columns
  const int head = blockIdx.y, batch = blockIdx.z;
  const int hidden = p.heads * kHeadDim;
#if HOM_DIAG_ENABLED
  const long long t_entry = clock64();
  long long *stamps = nullptr;
  if (p.prof != nullptr && tid == 0 && p.timeline_slot >= 0) {
    const long long now = static_cast<long long>(global_ns());
    atomicMin(p.prof + 32 + 4 * p.timeline_slot, now);
    atomicMax(p.prof + 33 + 4 * p.timeline_slot, now);
  } else if (p.prof != nullptr && tid == 0) {
    if (blockIdx.y == 0 && blockIdx.z == 0) stamps = p.prof;
    else if (blockIdx.y == gridDim.y / 2 && blockIdx.z == gridDim.z / 2) stamps = p.prof + 16;
  }
  // per-CTA wall-clock stamps of timeline launches 0 and 5: {entry, loaded, P written, exit}
  long long *cta_ns = nullptr;
  if (p.prof != nullptr && tid == 0 && (p.timeline_slot == 0 || p.timeline_slot == 5)) {
    const int cta = blockIdx.z * gridDim.y + blockIdx.y;
    if (cta < 448) cta_ns = p.prof + 64 + (p.timeline_slot == 5 ? 2016 : 0) + 4 * cta;
    if (cta_ns) cta_ns[0] = static_cast<long long>(global_ns());
  }
  auto stamp = [&](int slot) {
    if (stamps) stamps[slot] = clock64() - t_entry;
    if (cta_ns && slot == 3) cta_ns[1] = static_cast<long long>(global_ns());
    if (cta_ns && slot == 6) cta_ns[2] = static_cast<long long>(global_ns());
    if (cta_ns && slot == 9) cta_ns[3] = static_cast<long long>(global_ns());
  };
#else
  auto stamp = [](int) {};
#endif

  const uint32_t smem_q = smem_base, smem_k = smem_base + kTileBytes, smem_v = smem_base + 2 * kTileBytes;
  const uint32_t smem_p = smem_base;  // two 128 x 64 sub-tiles over Q|K
  const uint32_t bar_load = smem_base + 3 * kTileBytes;
  const uint32_t bar_s = bar_load + 8, bar_o = bar_load + 16;
  const uint32_t bar_v = bar_load + 32;  // V arrives on its own barrier: S and the softmax do not wait for it
  volatile uint32_t *tmem_slot = reinterpret_cast<volatile uint32_t *>(smem_gen + 3 * kTileBytes + 24);
  volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);
  float *xchg_max = reinterpret_cast<float *>(smem_gen + 3 * kTileBytes + 64);  // [2][128]
  float *xchg_sum = xchg_max + 2 * kTile;                                       // [2][128]

  if (tid == 0) {
    mbar_init(bar_load, 1);
    mbar_init(bar_v, 1);
    mbar_init(bar_s, 1);
    mbar_init(bar_o, 1);
    *abort_flag = 0;
    fence_mbar_init();
    prefetch_tensormap(&tmQKV);
    prefetch_tensormap(&tmOut);
  }
  if (warp == 0) {
    tmem_alloc(smem_u32(const_cast<uint32_t *>(tmem_slot)), 128);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_acc = *tmem_slot;
  // Dependents may be scheduled only now that every CTA of this grid holds its tensor memory.
  pdl_launch_dependents();
  const uint32_t lane_sel = static_cast<uint32_t>((warp & 3) * 32) << 16;
  stamp(0);

  pdl_wait();  // cu_seqlens and the packed QKV come from earlier kernels of the stream
  stamp(1);
  // The tiles do not depend on the valid length: request them before reading it.
  // Warp 0 runs the copy / MMA issue code as a whole (addresses and descriptors stay
  // warp-uniform); one elected lane executes the asynchronous instructions.
  const bool leader = warp == 0 && elect_one();
  if (leader) {
    const int row_base = batch * p.seq;
    mbar_arrive_expect_tx(bar_load, 2 * kTileBytes);
    tma_load_2d(smem_q, &tmQKV, bar_load, head * kHeadDim, row_base);
    tma_load_2d(smem_k, &tmQKV, bar_load, hidden + head * kHeadDim, row_base);
    mbar_arrive_expect_tx(bar_v, kTileBytes);
    tma_load_2d(smem_v, &tmQKV, bar_v, 2 * hidden + head * kHeadDim, row_base);
  }
  int len = p.cu_seqlens[batch + 1] - p.cu_seqlens[batch];
  len = max(0, min(len, p.seq));
  stamp(2);

  bool ok = true;
  float inv = 0.f;
  if (len > 0) {
    if (warp == 0) {
      if (__all_sync(0xffffffffu, mbar_wait(bar_load, 0, abort_flag, p.status, kDevWaitTimeoutAttention))) {
        stamp(3);
        tc_fence_after_sync();
        constexpr uint32_t idesc_s = make_idesc_f16(kTile, kTile, false, false);
#pragma unroll
        for (int k = 0; k < kHeadDim / 16; ++k) {
          const uint64_t da = make_smem_desc_sw128(smem_q + k * 32, 16, 1024);
          const uint64_t db = make_smem_desc_sw128(smem_k + k * 32, 16, 1024);
          if (leader) tc_mma_f16_ss(tmem_acc, da, db, idesc_s, k != 0 ? 1u : 0u);
        }
        if (leader) tc_commit(bar_s);
      }
    }
    ok = mbar_wait(bar_s, 0, abort_flag, p.status, kDevWaitTimeoutAttention);
    ok = __syncthreads_and(ok);
    stamp(4);
    if (ok) {
      tc_fence_after_sync();
      const bool row_live = row < len;  // padded query rows are written as zeros
      // tcgen05.ld is warp-collective: the whole warp takes part as soon as one of its rows is
      // live; what its padded rows compute is never used.
      const bool warp_live = (warp & 3) * 32 < len;
      const float2 scale2 = make_float2(p.scale_log2, p.scale_log2);
      // pass 1: maximum of this thread's scaled scores over the valid keys
      float m_part = -INFINITY;
      if (warp_live) {
#pragma unroll 1
        for (int c = 2 * hf; c < 2 * hf + 2 && c * 32 < len; ++c) {
          uint32_t r[32];
          tmem_ld_32x32(tmem_acc + lane_sel + c * 32, r);
          tmem_ld_wait();
          if ((c + 1) * 32 <= len) {
            float m0 = m_part, m1 = -INFINITY;
#pragma unroll
            for (int i = 0; i < 32; i += 2) {
              const float2 x = __fmul2_rn(make_float2(__uint_as_float(r[i]), __uint_as_float(r[i + 1])), scale2);
              m0 = fmaxf(m0, x.x);
              m1 = fmaxf(m1, x.y);
            }
            m_part = fmaxf(m0, m1);
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i)
              if (c * 32 + i < len) m_part = fmaxf(m_part, __uint_as_float(r[i]) * p.scale_log2);
          }
        }
      }
      xchg_max[hf * kTile + row] = m_part;
      __syncthreads();
      stamp(5);
      const float m_row = fmaxf(m_part, xchg_max[(hf ^ 1) * kTile + row]);
      // pass 2: P = exp2(s * scale - m) as fp16 into this thread's sub-tile row, and its sum
      float2 l2 = make_float2(0.f, 0.f);
      if (warp_live) {
        const float2 neg_m2 = make_float2(-m_row, -m_row);
        const uint32_t sub = smem_p + hf * kTileBytes + row * 128;
#pragma unroll 1
        for (int c = 2 * hf; c < 2 * hf + 2 && c * 32 < len; ++c) {
          uint32_t r[32];
          tmem_ld_32x32(tmem_acc + lane_sel + c * 32, r);
          tmem_ld_wait();
          const bool full = (c + 1) * 32 <= len;
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            uint32_t w[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const int i0 = g * 8 + 2 * j;
              const float2 x = __ffma2_rn(
                  make_float2(__uint_as_float(r[i0]), __uint_as_float(r[i0 + 1])), scale2, neg_m2);
              float2 e = make_float2(ex2_approx(x.x), ex2_approx(x.y));
              if (!full) {
                e.x = (c * 32 + i0 < len) ? e.x : 0.f;
                e.y = (c * 32 + i0 + 1 < len) ? e.y : 0.f;
              }
              l2 = __fadd2_rn(l2, e);
              const __half2 h = __floats2half2_rn(e.x, e.y);
              w[j] = *reinterpret_cast<const uint32_t *>(&h);
            }
            const uint32_t chunk = (c & 1) * 4 + g;
            const uint32_t addr = sub + ((chunk ^ (row & 7)) << 4);
            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(w[0]), "r"(w[1]),
                         "r"(w[2]), "r"(w[3])
                         : "memory");
          }
        }
      }
      const float l_part = l2.x + l2.y;
      xchg_sum[hf * kTile + row] = l_part;
      fence_proxy_async_smem();
      tc_fence_before_sync();
      __syncthreads();  // P complete, and every thread is done reading S
      stamp(6);
      const float l_row = l_part + xchg_sum[(hf ^ 1) * kTile + row];
      inv = (row_live && l_row > 0.f) ? 1.f / l_row : 0.f;
      if (warp == 0 &&
          __all_sync(0xffffffffu, mbar_wait(bar_v, 0, abort_flag, p.status, kDevWaitTimeoutAttention))) {
        tc_fence_after_sync();
        constexpr uint32_t idesc_o = make_idesc_f16(kTile, kHeadDim, false, true);
        const int k_steps = (len + 15) >> 4;  // key groups beyond the last valid key hold no P
        for (int k = 0; k < k_steps; ++k) {
          const uint64_t da =
              make_smem_desc_sw128(smem_p + (k >> 2) * kTileBytes + (k & 3) * 32, 16, 1024);
          const uint64_t db = make_smem_desc_sw128(smem_v + k * 2048, kTileBytes, 1024);
          if (leader) tc_mma_f16_ss(tmem_acc, da, db, idesc_o, k != 0 ? 1u : 0u);
        }
        if (leader) tc_commit(bar_o);
      }
      ok = mbar_wait(bar_o, 0, abort_flag, p.status, kDevWaitTimeoutAttention);
      ok = __syncthreads_and(ok);
      stamp(7);
    }
  }

  if (len == 0) {
    // Nothing was computed, but the tile copies are in flight: they must land before the
    // zero tile is staged over V (and before shared memory is released).
    ok = mbar_wait(bar_load, 0, abort_flag, p.status, kDevWaitTimeoutAttention);
    ok = ok && mbar_wait(bar_v, 0, abort_flag, p.status, kDevWaitTimeoutAttention);
    ok = __syncthreads_and(ok);
  }
  if (ok) {
    if (len > 0) tc_fence_after_sync();
    // O (or zeros for padded rows / empty sequences) -> swizzled staging over the V tile;
    // this thread owns output columns [32 * hf, +32) of its row.
    const uint32_t my_row = smem_v + row * 128;
    uint32_t r[32];
    if (len > 0) {  // block-uniform: the load is warp-collective
      tmem_ld_32x32(tmem_acc + lane_sel + hf * 32, r);
      tmem_ld_wait();
    }
    const float2 inv2 = make_float2(inv, inv);
#pragma unroll
    for (int g = 0; g < 4; ++g) {
      uint32_t w[4] = {0u, 0u, 0u, 0u};
      if (inv != 0.f) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 o = __fmul2_rn(make_float2(__uint_as_float(r[g * 8 + 2 * j]),
                                                  __uint_as_float(r[g * 8 + 2 * j + 1])), inv2);
          const __half2 h = __floats2half2_rn(o.x, o.y);
          w[j] = *reinterpret_cast<const uint32_t *>(&h);
        }
      }
      const uint32_t chunk = hf * 4 + g;
      const uint32_t addr = my_row + ((chunk ^ (row & 7)) << 4);
      asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(w[0]), "r"(w[1]),
                   "r"(w[2]), "r"(w[3])
                   : "memory");
    }
    fence_proxy_async_smem();
    tc_fence_before_sync();
    __syncthreads();
    stamp(8);
    if (leader) {
      asm volatile(
          "cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%2, %3, %4}], [%1];"
          :
          : "l"(reinterpret_cast<uint64_t>(&tmOut)), "r"(smem_v), "r"(head * kHeadDim), "r"(0),
            "r"(batch)
          : "memory");
      bulk_commit_group();
      bulk_wait_group_read_0();
      stamp(9);
    }
  } else if (tid == 0) {
    // Let copies that are still in flight land before the shared memory is released.
    const long long t0 = clock64();
    while (!mbar_try_wait(bar_load, 0) && clock64() - t0 < 200000000LL) {
    }
    while (!mbar_try_wait(bar_v, 0) && clock64() - t0 < 400000000LL) {
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_acc, 128);
  }
  HOM_DIAG(if (p.prof != nullptr && tid == 0 && p.timeline_slot >= 0) {
    const long long now = static_cast<long long>(global_ns());
    atomicMin(p.prof + 34 + 4 * p.timeline_slot, now);
    atomicMax(p.prof + 35 + 4 * p.timeline_slot, now);
  })
}

}  // namespace

namespace {

// Identity of a cached output tensor map: the whole (pointer, shape) tuple is compared, the
// hash only picks the bucket.
struct OutMapKey {
  const void *ptr;
  uint64_t hidden, seq, bs;
  bool operator==(const OutMapKey &o) const {
    return ptr == o.ptr && hidden == o.hidden && seq == o.seq && bs == o.bs;
  }
};
struct OutMapKeyHash {
  size_t operator()(const OutMapKey &k) const {
    size_t h = reinterpret_cast<size_t>(k.ptr);
    h = h * 1000003u ^ k.hidden;
    h = h * 1000003u ^ k.seq;
    h = h * 1000003u ^ k.bs;
    return h;
  }
};

// Output [bs, seq, hidden] fp16 as a 3-D tensor (hidden, seq, bs) with 64 x 128 x 1 boxes.
bool make_out_map(const void *ptr, uint64_t hidden, uint64_t seq, uint64_t bs, CUtensorMap *out) {
  static std::mutex mu;
  static std::unordered_map<OutMapKey, CUtensorMap, OutMapKeyHash> cache;
  const OutMapKey key{ptr, hidden, seq, bs};
  {
    std::lock_guard<std::mutex> lock(mu);
    auto it = cache.find(key);
    if (it != cache.end()) {
      *out = it->second;
      return true;
    }
  }
  using EncodeFn = CUresult (*)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *,
                                const cuuint64_t *, const cuuint64_t *, const cuuint32_t *,
                                const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
  void *sym = nullptr;
  cudaDriverEntryPointQueryResult qres;
  if (cudaGetDriverEntryPointByVersion("cuTensorMapEncodeTiled", &sym, 12000, cudaEnableDefault,
                                       &qres) != cudaSuccess ||
      qres != cudaDriverEntryPointSuccess) {
    set_error(HOM_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
    return false;
  }
  cuuint64_t dims[3] = {hidden, seq, bs};
  cuuint64_t strides[2] = {hidden * 2, hidden * seq * 2};
  cuuint32_t box[3] = {kHeadDim, kTile, 1};
  cuuint32_t elem[3] = {1, 1, 1};
  const CUresult r = reinterpret_cast<EncodeFn>(sym)(
      out, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, const_cast<void *>(ptr), dims, strides, box, elem,
      CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
      CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_error(HOM_ERR_CUDA, "cuTensorMapEncodeTiled (attention output) failed (%d)", static_cast<int>(r));
    return false;
  }
  std::lock_guard<std::mutex> lock(mu);
  if (cache.size() > 4096) cache.clear();
  cache.emplace(key, *out);
  return true;
}

}  // namespace

bool run(const Problem &pb, cudaStream_t stream) {
  if (pb.bs == 0 || pb.seq == 0 || pb.heads == 0) return true;
  // More than one KV tile: the two-query-tile kernel (it folds the positive softmax scale into
  // the row maximum; any other scale takes the general kernel below).
  if (pb.seq > kTile && pb.scale > 0.f HOM_DIAG(&& !std::getenv("HOM_ATTN_SERIAL"))) return run_pingpong(pb, stream);
  static bool attr_set[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !attr_set[dev]) {
    if (!check_cuda(cudaFuncSetAttribute(attention_f16_kernel,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes),
                    "cudaFuncSetAttribute(attention)"))
      return false;
    attr_set[dev] = true;
  }
  CUtensorMap tm;
  const uint64_t rows = static_cast<uint64_t>(pb.bs) * pb.seq;
  const uint64_t cols = 3ull * pb.heads * kHeadDim;
  if (!gemm::make_tensor_map_2d(pb.qkv, cols, rows, kHeadDim, kTile, &tm)) return false;
  const bool single_tile = pb.seq <= kTile;
  Params p;
  p.cu_seqlens = pb.cu_seqlens;
  p.out = pb.out;
  p.seq = static_cast<int>(pb.seq);
  p.heads = static_cast<int>(pb.heads);
  p.scale_log2 = pb.scale * 1.44269504088896340736f;
  p.status = device_status_word();
#if HOM_DIAG_ENABLED
  static const bool want_prof = std::getenv("HOM_ATTN_PROFILE") != nullptr;
  p.prof = nullptr;
  p.timeline_slot = -1;
  if (want_prof) {
    static int timeline_calls = 0;
    if (std::getenv("HOM_ATTN_TIMELINE")) {
      p.prof = gemm::profile_buffer_raw();
      p.timeline_slot = timeline_calls++ & 7;
    } else {
      p.prof = gemm::profile_buffer();
    }
  }
#endif
  dim3 grid(static_cast<unsigned>((pb.seq + kTile - 1) / kTile), static_cast<unsigned>(pb.heads),
            static_cast<unsigned>(pb.bs));
  const double d = kHeadDim;
  const double flops = 4.0 * d * pb.heads * pb.bs * static_cast<double>(pb.seq) * pb.seq;
  const double bytes = 2.0 * rows * cols + 2.0 * rows * pb.heads * d + 4.0 * (pb.bs + 1);
  LaunchScope scope(kOpAttention, flops, bytes);
  if (single_tile) {
    static bool attr1_set[64] = {};
    if (dev >= 0 && dev < 64 && !attr1_set[dev]) {
      if (!check_cuda(cudaFuncSetAttribute(attention_f16_single_tile_kernel,
                                           cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes1),
                      "cudaFuncSetAttribute(attention)"))
        return false;
      attr1_set[dev] = true;
    }
    CUtensorMap tm_out;
    if (!make_out_map(pb.out, pb.heads * kHeadDim, pb.seq, pb.bs, &tm_out)) return false;
    const bool launched = check_cuda(launch_pdl(attention_f16_single_tile_kernel, grid, dim3(kThreads1),
                                                kSmemBytes1, stream, 1, tm, tm_out, p),
                                     "attention kernel launch");
#if HOM_DIAG_ENABLED
    if (p.prof && p.timeline_slot < 0) {
      long long h[32];
      cudaStreamSynchronize(stream);
      cudaMemcpy(h, p.prof, sizeof(h), cudaMemcpyDeviceToHost);
      for (int c = 0; c < 2; ++c)
        fprintf(stderr,
                "[hom] attention CTA %s: setup %lld | dependency %lld | len %lld | loaded %lld | S %lld | "
                "max %lld | P %lld | O %lld | staged %lld | stored %lld cycles\n",
                c ? "mid" : "0", h[16 * c], h[16 * c + 1], h[16 * c + 2], h[16 * c + 3], h[16 * c + 4],
                h[16 * c + 5], h[16 * c + 6], h[16 * c + 7], h[16 * c + 8], h[16 * c + 9]);
    }
#endif
    return launched;
  }
  return check_cuda(launch_pdl(attention_f16_kernel, grid, dim3(kThreads), kSmemBytes, stream, 1, tm, p),
                    "attention kernel launch");
}

}  // namespace attention
}  // namespace hom
