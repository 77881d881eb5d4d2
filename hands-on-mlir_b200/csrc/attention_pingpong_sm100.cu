// Packed-QKV padded bidirectional attention for sequences longer than one 128-key tile,
// head_dim 64: a persistent, warp-specialised kernel in which one CTA owns TWO 128-row query
// tiles of one (batch, head) at a time so that the tensor pipe and the softmax arithmetic
// overlap: while the threads of tile A run their softmax on S_A, the tensor pipe computes
// P_B.V and S_B for tile B, and the other way round.
//
//   warp 0       TMA producer: the two Q tiles of a work item and a two-stage ring of K / V
//                tiles (128 x 64 fp16 boxes lifted out of the packed [bs*seq, 3*heads*64]
//                tensor into 128-byte-swizzled shared memory);
//   warp 1       issues every tcgen05.mma: S_t = Q_t.K_j^T (128 x 128 x 64) into the tile's S
//                columns of tensor memory and O_t = P_t.V_j (128 x 64 x 128) into its O
//                columns, and hands buffers on with tcgen05.commit;
//   warps 2-5    softmax of tile A, one query row per thread: row maximum and exponentials
//   warps 6-9    softmax of tile B  straight from tensor memory (two passes over S, fp32,
//                exp2 with the scale folded in), P written to shared memory as fp16 in the
//                K-major layout the second MMA reads, O_j folded into the running output in
//                registers with the online-softmax correction.
//
// Work items are (batch, head, pair of query tiles); a CTA walks items blockIdx.x,
// blockIdx.x + gridDim.x, ... and the K / V ring runs across item boundaries, so the loads of
// the next item overlap the arithmetic of the current one.  KV tiles beyond a sequence's valid
// length are skipped, the ragged tile is masked, query tiles that are all padding are not
// computed, and padded query rows are written as zeros.
//
// Same contract as the reference's cuDNN fused attention behind TransformerEngine
// (include/NVGPUKernels/BertAttentionRunner.h:52-136: layout BS3HD, no bias, padding mask,
// no dropout, inference).
#include <cstdio>
#include <cstdlib>

#include "attention_sm100.cuh"
#include "gemm_sm100.cuh"
#include "hom_diag.cuh"
#include "ptx_sm100.cuh"

namespace hom {
namespace attention {

using namespace hom::ptx;

namespace {

constexpr int kTile = 128;
constexpr int kHeadDim = 64;
constexpr uint32_t kTileBytes = kTile * kHeadDim * 2;  // 16 KB
constexpr int kThreadsPP = 320;                        // producer, MMA, 2 x 4 softmax warps
constexpr int kKvStages = 2;

// shared-memory map (offsets from the 1024-byte aligned base)
constexpr uint32_t kOffQ = 0;                                   // 2 tiles x 2 buffers (item i, item i + 1)
constexpr uint32_t kOffK = kOffQ + 4 * kTileBytes;              // kKvStages tiles
constexpr uint32_t kOffV = kOffK + kKvStages * kTileBytes;      // kKvStages tiles
constexpr uint32_t kOffP = kOffV + kKvStages * kTileBytes;      // 2 tiles x (two 128 x 64 sub-tiles)
constexpr uint32_t kOffBar = kOffP + 2 * 2 * kTileBytes;
constexpr uint32_t kSmemBytesPP = kOffBar + 256 + 1024;
// S_A, S_B: 128 columns each; O_A, O_B: two 64-column buffers each (the product of step j is
// folded into the running output while the tensor pipe already writes that of step j + 1)
constexpr uint32_t kTmemColsPP = 512;

struct ParamsPP {
  const int *cu_seqlens;
  __half *out;
  int seq, heads, bs;
  int q_pairs;    // pairs of query tiles per sequence = ceil(seq / 256)
  int num_items;  // bs * heads * q_pairs
  float scale_log2;
  int *status;
  HOM_DIAG(long long *prof;)  // phase cycle counters of CTA 0 (HOM_ATTN_PROFILE), else null
};

__device__ __forceinline__ float ex2_fast(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// What every role derives from an item number.
struct Item {
  int batch, head, q0;  // q0: first query row of tile A
  int len, n_kv;        // valid length, KV tiles that hold valid keys
  bool act[2];          // tile t has at least one valid query row
};

__device__ __forceinline__ Item decode_item(const ParamsPP &p, int item) {
  Item it;
  const int qp = item % p.q_pairs;
  const int bh = item / p.q_pairs;
  it.head = bh % p.heads;
  it.batch = bh / p.heads;
  it.q0 = qp * 2 * kTile;
  int len = p.cu_seqlens[it.batch + 1] - p.cu_seqlens[it.batch];
  len = max(0, min(len, p.seq));
  it.len = len;
  it.n_kv = (len + kTile - 1) / kTile;
  it.act[0] = it.q0 < len;
  it.act[1] = it.q0 + kTile < len;
  return it;
}

__global__ void __launch_bounds__(kThreadsPP, 1)
attention_f16_pingpong_kernel(const __grid_constant__ CUtensorMap tmQKV, const ParamsPP p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t smem_base = (raw_addr + 1023u) & ~1023u;
  uint8_t *smem_gen = smem_raw + (smem_base - raw_addr);

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;

  // barriers, 8 bytes each
  const uint32_t bar0 = smem_base + kOffBar;
  auto q_full = [&](int t, int b) { return bar0 + 8u * (2 * t + b); };        // Q_t buffer b loaded
  auto q_empty = [&](int t, int b) { return bar0 + 8u * (4 + 2 * t + b); };   // ... and consumed
  auto k_full = [&](int s) { return bar0 + 8u * (8 + s); };
  auto k_empty = [&](int s) { return bar0 + 8u * (10 + s); };
  auto v_full = [&](int s) { return bar0 + 8u * (12 + s); };
  auto v_empty = [&](int s) { return bar0 + 8u * (14 + s); };
  auto s_full = [&](int t) { return bar0 + 8u * (16 + t); };
  auto p_full = [&](int t) { return bar0 + 8u * (18 + t); };
  auto o_full = [&](int t, int b) { return bar0 + 8u * (20 + 2 * t + b); };   // O_t buffer b written
  auto o_empty = [&](int t, int b) { return bar0 + 8u * (24 + 2 * t + b); };  // ... and read
  volatile uint32_t *tmem_slot = reinterpret_cast<volatile uint32_t *>(smem_gen + kOffBar + 8 * 28);
  volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);

  if (tid == 64) prefetch_tensormap(&tmQKV);
  if (tid == 0) {
    for (int i = 0; i < 2; ++i) {
      mbar_init(k_full(i), 1);
      mbar_init(k_empty(i), 1);
      mbar_init(v_full(i), 1);
      mbar_init(v_empty(i), 1);
      mbar_init(s_full(i), 1);
      mbar_init(p_full(i), kTile);   // every softmax thread of the tile arrives
      for (int b = 0; b < 2; ++b) {
        mbar_init(q_full(i, b), 1);
        mbar_init(q_empty(i, b), 1);
        mbar_init(o_full(i, b), 1);
        mbar_init(o_empty(i, b), kTile);
      }
    }
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(const_cast<uint32_t *>(tmem_slot)), kTmemColsPP);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  // Dependents may be scheduled only now that this CTA holds its tensor memory.
  pdl_launch_dependents();
  pdl_wait();  // cu_seqlens and the packed QKV come from earlier kernels of the stream

  const int hidden = p.heads * kHeadDim;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    const bool leader = elect_one();
    uint32_t q_uses[2] = {0, 0};  // completed loads into each Q buffer
    uint32_t kv_uses = 0;         // K / V tiles loaded so far (stage = kv_uses % kKvStages)
    bool ok = true;
    for (int item = blockIdx.x; item < p.num_items && ok; item += gridDim.x) {
      const Item it = decode_item(p, item);
      if (!it.act[0]) continue;  // tile B cannot be active without tile A
      const int row_base = it.batch * p.seq;
      for (int t = 0; t < 2 && ok; ++t) {
        if (!it.act[t]) continue;
        // the buffer is free once every S MMA of the item that used it last has completed
        const int b = q_uses[t] & 1u;
        ok = __all_sync(0xffffffffu, mbar_wait(q_empty(t, b), ((q_uses[t] >> 1) & 1u) ^ 1u, abort_flag, p.status,
                                               kDevWaitTimeoutAttention));
        if (!ok) break;
        if (leader) {
          mbar_arrive_expect_tx(q_full(t, b), kTileBytes);
          tma_load_2d(smem_base + kOffQ + (2 * t + b) * kTileBytes, &tmQKV, q_full(t, b), it.head * kHeadDim,
                      row_base + it.q0 + t * kTile);
        }
        ++q_uses[t];
      }
      for (int j = 0; j < it.n_kv && ok; ++j) {
        const int s = kv_uses % kKvStages;
        const uint32_t ph = (kv_uses / kKvStages) & 1u;
        ok = __all_sync(0xffffffffu, mbar_wait(k_empty(s), ph ^ 1u, abort_flag, p.status, kDevWaitTimeoutAttention));
        if (!ok) break;
        if (leader) {
          mbar_arrive_expect_tx(k_full(s), kTileBytes);
          tma_load_2d(smem_base + kOffK + s * kTileBytes, &tmQKV, k_full(s), hidden + it.head * kHeadDim,
                      row_base + j * kTile);
        }
        ok = __all_sync(0xffffffffu, mbar_wait(v_empty(s), ph ^ 1u, abort_flag, p.status, kDevWaitTimeoutAttention));
        if (!ok) break;
        if (leader) {
          mbar_arrive_expect_tx(v_full(s), kTileBytes);
          tma_load_2d(smem_base + kOffV + s * kTileBytes, &tmQKV, v_full(s), 2 * hidden + it.head * kHeadDim,
                      row_base + j * kTile);
        }
        ++kv_uses;
      }
    }
    if (!ok) {
      // Give copies already in flight time to land before shared memory is released.
      const long long t0 = clock64();
      while (clock64() - t0 < 4000000LL) {
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------- MMA issuer
    // The whole warp runs the loop (addresses and descriptors stay warp-uniform); one elected
    // lane issues the MMAs and the commits.
    constexpr uint32_t idesc_s = make_idesc_f16(kTile, kTile, false, false);
    constexpr uint32_t idesc_o = make_idesc_f16(kTile, kHeadDim, false, true);
    const bool leader = elect_one();
    uint32_t q_uses[2] = {0, 0}, kv_uses = 0;
    uint32_t p_uses[2] = {0, 0}, o_uses[2] = {0, 0};
    bool ok = true;
    auto wait = [&](uint32_t bar, uint32_t parity) {
      ok = __all_sync(0xffffffffu, mbar_wait(bar, parity, abort_flag, p.status, kDevWaitTimeoutAttention));
      tc_fence_after_sync();
      return ok;
    };
    auto issue_s = [&](int t, int stage, int q_buf) {
      const uint32_t q_addr = smem_base + kOffQ + (2 * t + q_buf) * kTileBytes;
      const uint32_t k_addr = smem_base + kOffK + stage * kTileBytes;
#pragma unroll
      for (int k = 0; k < kHeadDim / 16; ++k) {
        const uint64_t da = make_smem_desc_sw128(q_addr + k * 32, 16, 1024);
        const uint64_t db = make_smem_desc_sw128(k_addr + k * 32, 16, 1024);
        if (leader) tc_mma_f16_ss(tmem_base + t * kTile, da, db, idesc_s, k != 0 ? 1u : 0u);
      }
      if (leader) tc_commit(s_full(t));
    };
    for (int item = blockIdx.x; item < p.num_items && ok; item += gridDim.x) {
      const Item it = decode_item(p, item);
      if (!it.act[0]) continue;
      const int n_act = it.act[1] ? 2 : 1;
      int qb[2] = {0, 0};
      for (int t = 0; t < n_act && ok; ++t) {
        qb[t] = q_uses[t] & 1u;
        wait(q_full(t, qb[t]), (q_uses[t] >> 1) & 1u);
        ++q_uses[t];
      }
      if (!ok) break;
      // S of the first KV tile for both query tiles
      {
        const int s = kv_uses % kKvStages;
        if (!wait(k_full(s), (kv_uses / kKvStages) & 1u)) break;
        for (int t = 0; t < n_act; ++t) issue_s(t, s, qb[t]);
        if (leader) tc_commit(k_empty(s));
      }
      for (int j = 0; j < it.n_kv && ok; ++j) {
        const int s = (kv_uses + j) % kKvStages;
        const uint32_t ph = ((kv_uses + j) / kKvStages) & 1u;
        const int valid = min(kTile, it.len - j * kTile);
        const int k_steps = (valid + 15) >> 4;  // key groups that hold a valid key
        const int s_next = (kv_uses + j + 1) % kKvStages;
        const uint32_t ph_next = ((kv_uses + j + 1) / kKvStages) & 1u;
        if (!wait(v_full(s), ph)) break;
        for (int t = 0; t < n_act && ok; ++t) {
          // P_t of this step is in shared memory and S_t has been read
          if (!wait(p_full(t), p_uses[t] & 1u)) break;
          ++p_uses[t];
          // S of the next KV tile first: the tile's threads need it before they need O
          if (j + 1 < it.n_kv) {
            if (t == 0 && !wait(k_full(s_next), ph_next)) break;
            issue_s(t, s_next, qb[t]);
            if (t == n_act - 1 && leader) tc_commit(k_empty(s_next));
          }
          // the O buffer this step writes was last read two steps ago
          const int ob = o_uses[t] & 1u;
          if (!wait(o_empty(t, ob), ((o_uses[t] >> 1) & 1u) ^ 1u)) break;
          ++o_uses[t];
          const uint32_t p_addr = smem_base + kOffP + t * 2 * kTileBytes;
          const uint32_t v_addr = smem_base + kOffV + s * kTileBytes;
          const uint32_t o_tmem = tmem_base + 2 * kTile + (2 * t + ob) * kHeadDim;
          for (int k = 0; k < k_steps; ++k) {
            const uint64_t da = make_smem_desc_sw128(p_addr + (k >> 2) * kTileBytes + (k & 3) * 32, 16, 1024);
            // V tile: 128 kv rows of 128 B; N (= d) contiguous, 16 kv rows = 2048 B.
            const uint64_t db = make_smem_desc_sw128(v_addr + k * 2048, kTileBytes, 1024);
            if (leader) tc_mma_f16_ss(o_tmem, da, db, idesc_o, k != 0 ? 1u : 0u);
          }
          if (leader) tc_commit(o_full(t, ob));
        }
        if (ok && leader) tc_commit(v_empty(s));
      }
      // every S MMA of the item has been issued: the Q buffers are free once they complete
      if (ok && leader) {
        for (int t = 0; t < n_act; ++t) tc_commit(q_empty(t, qb[t]));
      }
      kv_uses += it.n_kv;
    }
  } else {
    // ------------------------------------------------ softmax, one query row per thread
    const int t = (warp - 2) >> 2;             // which query tile of the pair
    const int quarter = warp & 3;              // the warp's tensor-memory lane quarter
    const int row = quarter * 32 + lane;       // row of the tile
    const uint32_t lane_sel = static_cast<uint32_t>(quarter * 32) << 16;
    const uint32_t tmem_s = tmem_base + t * kTile + lane_sel;
    const uint32_t tmem_o = tmem_base + 2 * kTile + 2 * t * kHeadDim + lane_sel;  // two buffers
    const uint32_t p_row = smem_base + kOffP + t * 2 * kTileBytes + row * 128;
    const float2 scale2 = make_float2(p.scale_log2, p.scale_log2);
    uint32_t s_uses = 0, o_uses = 0;
    bool ok = true;
    HOM_DIAG(long long c_wait_s = 0, c_pass1 = 0, c_pass2 = 0, c_wait_o = 0, c_fold = 0, c_store = 0, c_steps = 0;
             const long long c_begin = clock64(); long long c_t = 0;)
    for (int item = blockIdx.x; item < p.num_items && ok; item += gridDim.x) {
      const Item it = decode_item(p, item);
      const int q_idx = it.q0 + t * kTile + row;
      __half *out_row = p.out + (static_cast<long long>(it.batch) * p.seq + q_idx) * hidden + it.head * kHeadDim;
      if (!it.act[t]) {
        // the whole query tile is padding (or beyond the sequence): zeros
        if (q_idx < p.seq) {
          const uint4 z = make_uint4(0, 0, 0, 0);
#pragma unroll
          for (int g = 0; g < 8; ++g) reinterpret_cast<uint4 *>(out_row)[g] = z;
        }
        continue;
      }
      float m_run = -INFINITY, l_run = 0.f;
      float2 o_acc[32];
#pragma unroll
      for (int i = 0; i < 32; ++i) o_acc[i] = make_float2(0.f, 0.f);
      float corr_pending = 0.f;
      // o_acc <- o_acc * corr + (P.V of the oldest step not yet folded in)
      auto fold = [&](float corr) {
        HOM_DIAG(c_t = clock64();)
        const int ob = o_uses & 1u;
        ok = mbar_wait(o_full(t, ob), (o_uses >> 1) & 1u, abort_flag, p.status, kDevWaitTimeoutAttention);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) return false;
        ++o_uses;
        tc_fence_after_sync();
        HOM_DIAG(c_wait_o += clock64() - c_t; c_t = clock64();)
        const float2 corr2 = make_float2(corr, corr);
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          uint32_t r[32];
          tmem_ld_32x32(tmem_o + ob * kHeadDim + c * 32, r);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 16; ++i)
            o_acc[c * 16 + i] = __ffma2_rn(o_acc[c * 16 + i], corr2,
                                           make_float2(__uint_as_float(r[2 * i]), __uint_as_float(r[2 * i + 1])));
        }
        tc_fence_before_sync();
        mbar_arrive(o_empty(t, ob));
        HOM_DIAG(c_fold += clock64() - c_t;)
        return true;
      };

      for (int j = 0; j < it.n_kv && ok; ++j) {
        const int valid = min(kTile, it.len - j * kTile);  // columns [0, valid) are real keys
        HOM_DIAG(c_t = clock64();)
        ok = mbar_wait(s_full(t), s_uses & 1u, abort_flag, p.status, kDevWaitTimeoutAttention);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        ++s_uses;
        tc_fence_after_sync();
        HOM_DIAG(c_wait_s += clock64() - c_t; c_t = clock64(); ++c_steps;)
        // ---- pass 1: row maximum of scale * S over the valid keys
        float m_tile = -INFINITY;
#pragma unroll 1
        for (int c = 0; c < 4 && c * 32 < valid; ++c) {
          uint32_t r[32];
          tmem_ld_32x32(tmem_s + c * 32, r);
          tmem_ld_wait();
          if ((c + 1) * 32 <= valid) {
            float m0 = m_tile, m1 = -INFINITY;
#pragma unroll
            for (int i = 0; i < 32; i += 2) {
              m0 = fmaxf(m0, __uint_as_float(r[i]));
              m1 = fmaxf(m1, __uint_as_float(r[i + 1]));
            }
            m_tile = fmaxf(m0, m1);
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i)
              if (c * 32 + i < valid) m_tile = fmaxf(m_tile, __uint_as_float(r[i]));
          }
        }
        HOM_DIAG(c_pass1 += clock64() - c_t; c_t = clock64();)
        // scale > 0, so the maximum of the scaled scores is the scaled maximum
        const float m_new = fmaxf(m_run, m_tile * p.scale_log2);
        const float corr = ex2_fast(m_run - m_new);  // 0 on the first tile (m_run = -inf)
        // The tile's P buffer still holds the previous step's probabilities until that step's
        // P.V product has read them.  Its MMAs were queued right after this step's S, so they are
        // normally long done (the fold below waits for the same phase), but nothing else orders
        // them before the stores of pass 2: a short pass 1 (a ragged last KV tile with a few
        // valid keys) can get here first.
        if (j > 0) {
          ok = mbar_wait(o_full(t, o_uses & 1u), (o_uses >> 1) & 1u, abort_flag, p.status, kDevWaitTimeoutAttention);
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
        }
        // ---- pass 2: P = exp2(scale * S - m) as fp16 into shared memory, row sum in fp32
        float2 l2 = make_float2(0.f, 0.f);
        const float2 neg_m2 = make_float2(-m_new, -m_new);
#pragma unroll 1
        for (int c = 0; c < 4; ++c) {
          const uint32_t sub = p_row + (c >> 1) * kTileBytes;
          // Chunks that lie entirely beyond the valid keys are never read by the second MMA
          // (it stops at the last 16-key group that holds a valid key).
          if (c * 32 >= valid) break;
          uint32_t r[32];
          tmem_ld_32x32(tmem_s + c * 32, r);
          tmem_ld_wait();
          const bool full = (c + 1) * 32 <= valid;
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            uint32_t w[4];
#pragma unroll
            for (int jj = 0; jj < 4; ++jj) {
              const int i0 = g * 8 + 2 * jj;
              const float2 x = __ffma2_rn(make_float2(__uint_as_float(r[i0]), __uint_as_float(r[i0 + 1])), scale2,
                                          neg_m2);
              float2 e = make_float2(ex2_fast(x.x), ex2_fast(x.y));
              if (!full) {
                e.x = (c * 32 + i0 < valid) ? e.x : 0.f;
                e.y = (c * 32 + i0 + 1 < valid) ? e.y : 0.f;
              }
              l2 = __fadd2_rn(l2, e);
              const __half2 h = __floats2half2_rn(e.x, e.y);
              w[jj] = *reinterpret_cast<const uint32_t *>(&h);
            }
            const uint32_t chunk = (c & 1) * 4 + g;
            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(sub + ((chunk ^ (row & 7)) << 4)),
                         "r"(w[0]), "r"(w[1]), "r"(w[2]), "r"(w[3])
                         : "memory");
          }
        }
        l_run = fmaf(l_run, corr, l2.x + l2.y);
        m_run = m_new;
        // P is complete and S has been read: hand both to the MMA warp
        fence_proxy_async_smem();
        tc_fence_before_sync();
        mbar_arrive(p_full(t));
        HOM_DIAG(c_pass2 += clock64() - c_t;)
        // ---- the product of the PREVIOUS step is folded in now: its MMA had this step's whole
        // softmax to finish, and the tensor pipe is already busy with this step's product
        if (j > 0 && !fold(corr_pending)) break;
        corr_pending = corr;
      }
      if (!ok) break;
      if (!fold(corr_pending)) break;
      if (!ok) break;
      HOM_DIAG(c_t = clock64();)
      if (q_idx < p.seq) {
        const bool real_row = q_idx < it.len && l_run > 0.f;
        const float inv = real_row ? 1.f / l_run : 0.f;
        const float2 inv2 = make_float2(inv, inv);
#pragma unroll
        for (int g = 0; g < 8; ++g) {
          uint4 o = make_uint4(0, 0, 0, 0);
          if (real_row) {
            __half2 *o2 = reinterpret_cast<__half2 *>(&o);
#pragma unroll
            for (int jj = 0; jj < 4; ++jj) {
              const float2 v = __fmul2_rn(o_acc[g * 4 + jj], inv2);
              o2[jj] = __floats2half2_rn(v.x, v.y);
            }
          }
          reinterpret_cast<uint4 *>(out_row)[g] = o;
        }
      }
      HOM_DIAG(c_store += clock64() - c_t;)
    }
    HOM_DIAG(if (p.prof && blockIdx.x == 0 && lane == 0 && (warp == 2 || warp == 6)) {
      long long *o = p.prof + (warp == 2 ? 0 : 8);
      o[0] = clock64() - c_begin; o[1] = c_wait_s; o[2] = c_pass1; o[3] = c_pass2; o[4] = c_wait_o; o[5] = c_fold;
      o[6] = c_store; o[7] = c_steps;
    })
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, kTmemColsPP);
  }
}

}  // namespace

bool run_pingpong(const Problem &pb, cudaStream_t stream) {
  static bool attr_set[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !attr_set[dev]) {
    if (!check_cuda(cudaFuncSetAttribute(attention_f16_pingpong_kernel,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytesPP),
                    "cudaFuncSetAttribute(attention, two query tiles per CTA)"))
      return false;
    attr_set[dev] = true;
  }
  CUtensorMap tm;
  const uint64_t rows = static_cast<uint64_t>(pb.bs) * pb.seq;
  const uint64_t cols = 3ull * pb.heads * kHeadDim;
  if (!gemm::make_tensor_map_2d(pb.qkv, cols, rows, kHeadDim, kTile, &tm)) return false;
  ParamsPP p;
  p.cu_seqlens = pb.cu_seqlens;
  p.out = pb.out;
  p.seq = static_cast<int>(pb.seq);
  p.heads = static_cast<int>(pb.heads);
  p.bs = static_cast<int>(pb.bs);
  p.q_pairs = static_cast<int>((pb.seq + 2 * kTile - 1) / (2 * kTile));
  const int64_t items = pb.bs * pb.heads * p.q_pairs;
  if (items > INT32_MAX) {
    set_error(HOM_ERR_UNSUPPORTED, "attention: too many (batch, head, query tile) work items");
    return false;
  }
  p.num_items = static_cast<int>(items);
  p.scale_log2 = pb.scale * 1.44269504088896340736f;
  p.status = device_status_word();
  HOM_DIAG(p.prof = std::getenv("HOM_ATTN_PROFILE") ? gemm::profile_buffer() : nullptr;)
  const int grid = p.num_items < sm_count() ? p.num_items : sm_count();
  const double d = kHeadDim;
  const double flops = 4.0 * d * pb.heads * pb.bs * static_cast<double>(pb.seq) * pb.seq;
  const double bytes = 2.0 * rows * cols + 2.0 * rows * pb.heads * d + 4.0 * (pb.bs + 1);
  LaunchScope scope(kOpAttention, flops, bytes);
  const bool launched = check_cuda(launch_pdl(attention_f16_pingpong_kernel, dim3(grid), dim3(kThreadsPP),
                                              kSmemBytesPP, stream, 1, tm, p),
                                   "attention kernel launch");
#if HOM_DIAG_ENABLED
  if (p.prof) {
    long long h[16];
    cudaStreamSynchronize(stream);
    cudaMemcpy(h, p.prof, sizeof(h), cudaMemcpyDeviceToHost);
    for (int w = 0; w < 2; ++w)
      fprintf(stderr,
              "[hom] attention CTA 0 tile %c: total %lld | wait S %lld | pass 1 %lld | pass 2 %lld | wait O %lld | "
              "fold %lld | store %lld cycles over %lld steps\n",
              w ? 'B' : 'A', h[8 * w], h[8 * w + 1], h[8 * w + 2], h[8 * w + 3], h[8 * w + 4], h[8 * w + 5],
              h[8 * w + 6], h[8 * w + 7]);
  }
#endif
  return launched;
}

}  // namespace attention
}  // namespace hom
