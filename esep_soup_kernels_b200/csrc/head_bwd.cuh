// Backward sweep of the LM head: dHidden = ce_weight * (softmax(x W^T) - onehot(target)) W,
// with the logits recomputed tile by tile and never written to global memory.
//
// Replaces, for all rows, the reference's per-chunk sequence
//     head_row_softmax_kernel pass 2: g = (e^(z-lse) - onehot) * G_SCALE   (kernels.py:84-93)
//     torch.mm(g, W, out_dtype=fp32) ; dx *= ce_weight / G_SCALE           (op.py:99-100)
//
// Geometry. A 128-row x H fp32 accumulator does not fit the 512 TMEM columns of one SM, so a
// cluster of 4 CTAs owns one 128-row tile of x and CTA c accumulates the H-slice
// [hs0, hs0 + 128*NHB) of dHidden (NHB <= 3 blocks of 128 TMEM columns; H = 1536 -> 4 x 384).
// Both GEMMs are computed TRANSPOSED so that the 128 token rows are the MMA N dimension, and the
// four CTAs work as two CTA pairs (cta_group::2, M = 256): the two CTAs of a pair then each hold
// only HALF of every B operand (64 token rows), which halves the x traffic and the P buffer and
// keeps shared-memory reads at 96 B/clk per SM. Per step the cluster covers 512 vocabulary rows:
//   G1  S^T[v, r] = W[vblock_c, :] . x[r, :]^T     A = W block (K-major), B = x half (K-major)
//       CTA c gets the 128 vocabulary rows of block c on its 128 TMEM lanes.
//   EPI thread = vocabulary row: p = e^(S - lse[r]) scaled and rounded to 16 bit, written as one
//       128-byte line per v (MN-major 128-byte-swizzle layout) per 64-row half. The half this
//       CTA consumes itself goes straight into its own P buffer, the other half into a 16 KiB
//       staging area; three asynchronous bulk copies (cp.async.bulk shared::cta ->
//       shared::cluster, 16 KiB each) then deliver the halves to the three other CTAs, counted
//       on the receivers' per-block mbarriers; a CTA may refill its block of every P buffer as
//       soon as both pairs' MMAs on that block have retired, while the G2 stream still works on
//       the later blocks of the step. (Per-lane remote stores were measured 6x slower.)
//   G2  dX^T[h, r] += sum_v W[v, h] P[v, r]        A = W tile (MN-major), B = P half (MN-major)
// The -onehot(target) term is applied in fp32 when the accumulator is drained:
// dX[r, :] -= ce_weight[r] * W[target[r], :]  (once, by the work unit that owns the target).
// G1 and G2 are two independent streams: each has its own TMA producer warp, its own ring of
// shared-memory slots and its own issuing warp, and the tensor pipe takes MMAs from whichever
// stream has work (tcgen05.mma blocks its issuer while the pipe is busy and the pipe queues
// almost nothing, so a single issuer that waits on a barrier idles the pipe). The streams are
// only tied by data: G1(s+1) needs the logits tile of step s drained, G2(s) needs P(s).
//
// Warp roles (256 threads): warp 0 = G1 producer, warp 1 = G1 issuer (pair leader) + TMEM owner,
// warp 2 = G2 producer, warp 3 = G2 issuer (pair leader) / P-barrier relay (pair peer),
// warps 4..7 = epilogue.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "head_fwd.cuh"

namespace esep {

enum : int {
  DEV_TIMEOUT_BWD_PRODUCER = 201,
  DEV_TIMEOUT_BWD_MMA = 202,
  DEV_TIMEOUT_BWD_EPILOGUE = 203,
};

struct BwdParams {
  int n, h, v;
  int n_row_tiles;      // ceil(n / 128)
  int nhb;              // 128-wide H blocks per CTA (1..3); H-slice per CTA = 128 * nhb
  int n_passes;         // ceil(h / (4 * 128 * nhb)): each pass recomputes the logits once
  int total_steps;      // ceil(ceil(v / 128) / 4)
  int full_rounds;        // rounds in which every cluster sweeps one whole (row tile, pass)
  int rem_tp;             // (row tile, pass) pairs left over after the full rounds
  int rem_splits;         // vocabulary runs each left-over pair is cut into (0 if none)
  int steps_per_split;    // steps per such run
  float* dx_part;         // [rem_splits, rem_tp * 128 rows, pass width] partial sums of those
  long long vocab_offset;
  const long long* target;  // [n] global ids
  const float* cew;         // [n] ce_weight, already zero on ignored rows
  const float* lse;         // [n] log-sum-exp over the FULL vocabulary
  const void* w;            // [v, h] 16-bit, for the onehot term
  float* dx;                // [n, h]
  float p_scale;            // 1024 for fp16 P (keeps 1/V out of the subnormals), 1 for bf16
  int w2_is_3d;             // tmap_w2 is the 3-D view {64 h, v, h / 64} (h % 64 == 0)
  int* status;
  const int* gate;          // null, or a device flag: the kernel does nothing when it reads 0
};

namespace bwd {
static constexpr int CL = 4;            // CTAs per cluster
static constexpr int BM = 128;          // token rows per cluster (MMA N)
static constexpr int BV = 128;          // vocabulary rows per CTA per step (TMEM lanes)
static constexpr int STEP_V = CL * BV;  // vocabulary rows per cluster per step
static constexpr int BK = 64;
static constexpr int SLOTS_A = 3;             // ring of the G1 stream
static constexpr int SLOTS_B = 3;             // ring of the G2 stream
static constexpr int SLOTS = SLOTS_A + SLOTS_B;
static constexpr int SLOT_BYTES = 24576;      // G1: W 128x64 (16 KiB) + x 64x64 (8 KiB)
static constexpr int G2_KV = 32;              // G2: 32 vocabulary rows x 384 h (6 boxes of 4 KiB)
static constexpr int P_BYTES = STEP_V * 128;  // [512 v][64 rows] 16-bit = 64 KiB
static constexpr int HALF_BYTES = BV * 128;   // one CTA's block for one 64-row half = 16 KiB
static constexpr int STAGE_BYTES = HALF_BYTES;
static constexpr int THREADS = 256;
static constexpr int TMEM_COLS = 512;
static constexpr int S_COL = 384;  // logits tile lives in TMEM columns [384, 512)
static constexpr int KC_PER_BLOCK = BV / G2_KV;   // G2 K-chunks per 128-row vocabulary block
// barriers: full[6] empty[6] (slots 0..2 G1 ring, 3..5 G2 ring) s_full s_empty p_empty
//           dx_full dx_empty rd_ready rd_free stage_ready p_in[4] p_peer[4]
static constexpr int NUM_BARS = 2 * SLOTS + 8 + 2 * CL;
static constexpr int ROWDATA_BYTES = 3 * BM * 4;  // per-row c2[128], rs[128], target-local[128]
static constexpr int SMEM_BYTES =
    1024 + P_BYTES + STAGE_BYTES + SLOTS * SLOT_BYTES + NUM_BARS * 8 + 64 + 16 + ROWDATA_BYTES;
static_assert(SMEM_BYTES <= 232448, "exceeds the 227 KiB of shared memory a CTA may use");
}  // namespace bwd

// Work split of the clustered sweeps. `n_tp` (row tile, pass) pairs go to `ncl` clusters:
//  1. full rounds: in round r cluster k sweeps pair r * ncl + k through the whole vocabulary;
//  2. the rem_tp < ncl left-over pairs are each cut into rem_splits vocabulary runs of
//     steps_per_split steps, so that (almost) every cluster gets one run.
// Pure integer arithmetic shared by the host plan and by kernels that learn their row count on
// the device.
struct SweepSplit {
  int full_rounds, rem_tp, rem_splits, steps_per_split;
};
__host__ __device__ inline SweepSplit sweep_split(long long n_tp, int ncl, int total_steps) {
  SweepSplit r;
  if (ncl < 1) ncl = 1;
  r.full_rounds = static_cast<int>(n_tp / ncl);
  r.rem_tp = static_cast<int>(n_tp - static_cast<long long>(r.full_rounds) * ncl);
  r.rem_splits = 0;
  r.steps_per_split = 0;
  if (r.rem_tp > 0 && total_steps > 0) {
    int want = ncl / r.rem_tp;
    if (want > total_steps) want = total_steps;
    if (want < 1) want = 1;
    r.steps_per_split = (total_steps + want - 1) / want;
    r.rem_splits = (total_steps + r.steps_per_split - 1) / r.steps_per_split;
  }
  return r;
}

template <int kFmt>
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
  if (kFmt == 0) {
    __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&h);
  } else {
    __nv_bfloat162 b = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&b);
  }
}

template <int kFmt>
__device__ __forceinline__ float load16(const void* base, size_t idx) {
  if (kFmt == 0) return __half2float(reinterpret_cast<const __half*>(base)[idx]);
  return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(base)[idx]);
}

template <int kFmt>
__global__ void __launch_bounds__(bwd::THREADS, 1)
head_bwd_kernel(const __grid_constant__ CUtensorMap tmap_x,    // x [n, h], box {64 k, 64 rows}
                const __grid_constant__ CUtensorMap tmap_w1,   // W [v, h], box {64 k, 128 v}
                const __grid_constant__ CUtensorMap tmap_w2,   // W as {64 h, v, h/64}, box {64, 32, 6}
                                                               // (or 2-D, box {64 h, 32 v})
                const BwdParams p) {
  using namespace bwd;
  if (p.gate != nullptr && *p.gate == 0) return;   // guarded launch: not needed this time
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* gen_base = smem_raw + (base - raw);
  const uint32_t p_base = base;                       // P buffer of this CTA (its 64 rows)
  const uint32_t stage_buf = base + P_BYTES;          // the 64-row half other CTAs consume
  const uint32_t ring = stage_buf + STAGE_BYTES;
  const uint32_t bars = ring + SLOTS * SLOT_BYTES;
  auto ring_full = [&](int s) { return bars + 8u * s; };
  auto ring_empty = [&](int s) { return bars + 8u * (SLOTS + s); };
  const uint32_t s_full = bars + 8u * (2 * SLOTS + 0);
  const uint32_t s_empty = bars + 8u * (2 * SLOTS + 1);
  const uint32_t p_empty = bars + 8u * (2 * SLOTS + 2);
  const uint32_t dx_full = bars + 8u * (2 * SLOTS + 3);
  const uint32_t dx_empty = bars + 8u * (2 * SLOTS + 4);
  const uint32_t rd_ready = bars + 8u * (2 * SLOTS + 5);
  const uint32_t rd_free = bars + 8u * (2 * SLOTS + 6);
  const uint32_t stage_ready = bars + 8u * (2 * SLOTS + 7);
  // One barrier per 128-row vocabulary block of the P buffer (block b is produced by CTA b):
  // p_in(b): block b of this CTA's buffer holds the current step; p_peer(b) (leader only): the
  // pair peer's buffer does too.
  auto p_in = [&](uint32_t b) { return bars + 8u * (2 * SLOTS + 8 + b); };
  auto p_peer = [&](uint32_t b) { return bars + 8u * (2 * SLOTS + 8 + CL + b); };
  const int misc_off = P_BYTES + STAGE_BYTES + SLOTS * SLOT_BYTES + NUM_BARS * 8;
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(gen_base + misc_off);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(gen_base + misc_off + 8);
  float* row_data = reinterpret_cast<float*>(gen_base + ((misc_off + 64 + 15) & ~15));  // float4 reads

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t c = cluster_ctarank();     // 0..3: vocabulary block and H-slice of this CTA
  const uint32_t leader = c & ~1u;          // pair leader rank
  const bool is_leader = (c == leader);
  const uint32_t half = c & 1u;             // which 64 token rows this CTA feeds as B operand
  const uint16_t pair_mask = static_cast<uint16_t>(3u << leader);
  const int cluster_id = blockIdx.x / CL;
  const int kblocks = (p.h + BK - 1) / BK;
  // Work decomposition. Tiles are (row tile, pass) pairs "tp" of total_steps steps each.
  //  1. full rounds: in round r cluster k sweeps tp = r * n_clusters + k from step 0 to the
  //     end and writes dHidden directly;
  //  2. the rem_tp < n_clusters left-over tiles are each cut into rem_splits vocabulary runs so
  //     that (almost) every cluster gets one run: cluster k < rem_tp * rem_splits takes run
  //     k / rem_tp of tile k % rem_tp and writes a partial piece (head_dx_sum_kernel adds them).
  // In both phases concurrently running clusters work on the same few vocabulary positions, so
  // W tiles are shared through L2 and come from HBM about once per sweep.
  // A cluster walks a private position axis u: [0, full_len) for the rounds, then one more
  // position for its left-over run.
  const int n_clusters = gridDim.x / CL;
  const long long full_len = static_cast<long long>(p.full_rounds) * p.total_steps;
  const bool has_rem = cluster_id < p.rem_tp * p.rem_splits;
  const long long u_first = (full_len > 0 || has_rem) ? 0 : 1;
  const long long u_last = full_len + (has_rem ? 1 : 0);
  const int hs = p.nhb * 128;

  if (threadIdx.x == 0) {
    for (int s = 0; s < SLOTS; ++s) {
      mbar_init(ring_full(s), 1);    // leader's producer arrive + bytes of both CTAs
      mbar_init(ring_empty(s), 1);   // one pair commit
    }
    mbar_init(s_full, 1);            // pair commit
    mbar_init(s_empty, 2 * 4);       // epilogue warps of both CTAs (leader's barrier)
    for (uint32_t b = 0; b < CL; ++b) {
      // own block: the four epilogue warps that write it; other blocks: the arming arrive (+ 16 KiB)
      mbar_init(p_in(b), b == c ? 4 : 1);
      mbar_init(p_peer(b), 1);       // relay arrive from the pair peer
    }
    mbar_init(rd_free, 4);           // epilogue warps of this CTA
    mbar_init(stage_ready, 4);       // epilogue warps of this CTA
    mbar_init(p_empty, 2);           // one commit per pair, after THIS CTA's block is consumed
    mbar_init(dx_full, 1);           // pair commit
    mbar_init(dx_empty, 2 * 4);      // epilogue warps of both CTAs (leader's barrier)
    mbar_init(rd_ready, 128);        // epilogue threads of this CTA
    *abort_flag = 0;
    fence_barrier_init();
    fence_proxy_async();
    tma_prefetch_desc(&tmap_x);
    tma_prefetch_desc(&tmap_w1);
    tma_prefetch_desc(&tmap_w2);
  }
  if (warp == 1) {
    tmem_alloc_pair(smem_u32(const_cast<uint32_t*>(tmem_slot)), TMEM_COLS);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  cluster_arrive();  // peers must see initialised barriers before any remote arrive / store
  cluster_wait();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  auto unit_tp = [&](long long u) {
    return u < full_len ? static_cast<int>(u / p.total_steps) * n_clusters + cluster_id
                        : p.full_rounds * n_clusters + cluster_id % p.rem_tp;
  };
  auto unit_rt = [&](long long u) { return unit_tp(u) % p.n_row_tiles; };
  auto unit_pass = [&](long long u) { return unit_tp(u) / p.n_row_tiles; };
  auto unit_steps = [&](long long u, int& s0, int& s1) {  // unit that starts at position u
    if (u < full_len) {
      s0 = 0;
      s1 = p.total_steps;
    } else {
      s0 = (cluster_id / p.rem_tp) * p.steps_per_split;
      s1 = min(p.total_steps, s0 + p.steps_per_split);
    }
  };
  auto unit_next = [&](long long u) { return u < full_len ? u + p.total_steps : u + 1; };

  if (warp == 0) {
    // ------------------- G1 producer (every CTA; whole warp, one lane issues) -----------
    // Ring slots 0 .. SLOTS_A-1: W block k-slice (16 KiB) + x half k-slice (8 KiB).
    const bool elected = elect_one_sync();
    uint32_t stage = 0, phase = 0;
    bool ok = true;
    const uint32_t full_leader0 = mapa_shared(ring_full(0), leader);
    for (long long u = u_first; u < u_last && ok; u = unit_next(u)) {
      const int xrow = unit_rt(u) * BM + static_cast<int>(half) * 64;
      int s0, s1;
      unit_steps(u, s0, s1);
      for (int step = s0; step < s1 && ok; ++step) {
        const int vrow = (step * CL + static_cast<int>(c)) * BV;
        for (int kb = 0; kb < kblocks; ++kb) {
          ok = mbar_wait_warp<true>(ring_empty(stage), phase ^ 1u, abort_flag);
          if (!ok) break;
          if (elected) {
            // the leader's barrier counts the bytes of both CTAs
            if (is_leader) mbar_expect_tx(ring_full(stage), 2 * SLOT_BYTES);
            const uint32_t sa = ring + stage * SLOT_BYTES;
            const uint32_t bar = full_leader0 + 8u * stage;
            tma_load_2d_pair(sa, &tmap_w1, bar, kb * BK, vrow);
            tma_load_2d_pair(sa + 16384, &tmap_x, bar, kb * BK, xrow);
          }
          if (++stage == SLOTS_A) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
    }
    if (!ok && elected) {
      *abort_flag = 1;
      atomicCAS(p.status, DEV_OK, DEV_TIMEOUT_BWD_PRODUCER);
    }
  } else if (warp == 2) {
    // ------------------- G2 producer (every CTA; whole warp, one lane issues) -----------
    // Ring slots SLOTS_A .. SLOTS-1: W[32 vocabulary rows, this CTA's 384 h] (24 KiB).
    const bool elected = elect_one_sync();
    uint32_t stage = 0, phase = 0;
    bool ok = true;
    const uint32_t full_leader0 = mapa_shared(ring_full(SLOTS_A), leader);
    for (long long u = u_first; u < u_last && ok; u = unit_next(u)) {
      const int hs0 = (unit_pass(u) * CL + static_cast<int>(c)) * hs;
      int s0, s1;
      unit_steps(u, s0, s1);
      for (int step = s0; step < s1 && ok; ++step) {
        for (int kc = 0; kc < STEP_V / G2_KV; ++kc) {
          ok = mbar_wait_warp<true>(ring_empty(SLOTS_A + stage), phase ^ 1u, abort_flag);
          if (!ok) break;
          if (elected) {
            if (is_leader) mbar_expect_tx(ring_full(SLOTS_A + stage), 2 * SLOT_BYTES);
            const uint32_t sa = ring + (SLOTS_A + stage) * SLOT_BYTES;
            const uint32_t bar = full_leader0 + 8u * stage;
            const int vrow = step * STEP_V + kc * G2_KV;
            if (p.w2_is_3d) {
              // one 24 KiB request: 6 blocks of 64 h x 32 v; blocks past h / 64 read zeros
              tma_load_3d_pair(sa, &tmap_w2, bar, 0, vrow, hs0 / 64);
            } else {
#pragma unroll
              for (int b = 0; b < 6; ++b)   // always 6 boxes: blocks beyond the slice read zeros
                tma_load_2d_pair(sa + b * 4096, &tmap_w2, bar,
                                 b < 2 * p.nhb ? hs0 + b * 64 : p.h + 64, vrow);
            }
          }
          if (++stage == SLOTS_B) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
    }
    if (!ok && elected) {
      *abort_flag = 1;
      atomicCAS(p.status, DEV_OK, DEV_TIMEOUT_BWD_PRODUCER);
    }
  } else if (warp == 1) {
    // ------------------- G1 issuer (pair leader only; whole warp, one lane issues) ------
    if (is_leader) {
      const bool elected = elect_one_sync();
      constexpr uint32_t idesc1 = make_idesc(kFmt, 256, BM, 0, 0);  // K-major A and B
      uint32_t stage = 0, phase = 0, g1par = 0;
      bool ok = true;
      const uint32_t d = tmem_base + S_COL;
      for (long long u = u_first; u < u_last && ok; u = unit_next(u)) {
        int s0, s1;
        unit_steps(u, s0, s1);
        for (int step = s0; step < s1 && ok; ++step) {
          // both epilogues must have pulled the previous logits tile out of TMEM
          ok = mbar_wait_warp<true>(s_empty, g1par ^ 1u, abort_flag);
          if (!ok) break;
          tc_fence_after();
          for (int kb = 0; kb < kblocks; ++kb) {
            ok = mbar_wait_warp<true>(ring_full(stage), phase, abort_flag);
            if (!ok) break;
            tc_fence_after();
            const uint32_t sa = ring + stage * SLOT_BYTES;
            const uint64_t adesc = make_smem_desc(sa, 16, 1024);          // W block, 128 v rows
            const uint64_t bdesc = make_smem_desc(sa + 16384, 16, 1024);  // x half, 64 rows
            if (elected) {
              umma_f16_ss_pair(d, adesc, bdesc, idesc1, kb != 0);
              umma_f16_ss_pair(d, adesc + 2u, bdesc + 2u, idesc1, 1u);
              umma_f16_ss_pair(d, adesc + 4u, bdesc + 4u, idesc1, 1u);
              umma_f16_ss_pair(d, adesc + 6u, bdesc + 6u, idesc1, 1u);
              umma_commit_pair_mask(ring_empty(stage), pair_mask);
            }
            if (++stage == SLOTS_A) {
              stage = 0;
              phase ^= 1u;
            }
          }
          if (ok && elected) umma_commit_pair_mask(s_full, pair_mask);
          g1par ^= 1u;
        }
      }
      if (!ok && elected) {
        *abort_flag = 1;
        atomicCAS(p.status, DEV_OK, DEV_TIMEOUT_BWD_MMA);
      }
    }
  } else if (warp == 3) {
    if (is_leader) {
      // ----------------- G2 issuer (pair leader; whole warp, one lane issues) -----------
      const bool elected = elect_one_sync();
      constexpr uint32_t idesc2 = make_idesc(kFmt, 256, BM, 1, 1);  // MN-major A and B
      uint32_t stage = 0, phase = 0, g2par = 0, upar = 0;
      bool ok = true;
      if (elected)   // first step: 16 KiB from each of the three other CTAs
        for (uint32_t b = 0; b < CL; ++b)
          if (b != c) mbar_expect_tx(p_in(b), HALF_BYTES);
      for (long long u = u_first; u < u_last && ok; u = unit_next(u)) {
        int s0, s1;
        unit_steps(u, s0, s1);
        for (int step = s0; step < s1 && ok; ++step) {
          // B = P half: one 128-byte line per vocabulary row, 8-row groups 1024 B apart.
          uint64_t bdesc = make_smem_desc(p_base, 8192, 1024);
          uint32_t acc0 = (step == s0) ? 0u : 1u;
          for (int kc = 0; kc < STEP_V / G2_KV; ++kc) {
            if ((kc & (KC_PER_BLOCK - 1)) == 0) {
              // block b of P (from CTA b) must be in this CTA's buffer and in the peer's
              const uint32_t b = static_cast<uint32_t>(kc / KC_PER_BLOCK);
              ok = mbar_wait_warp<true>(p_in(b), g2par, abort_flag) &&
                   mbar_wait_warp<true>(p_peer(b), g2par, abort_flag);
              if (!ok) break;
              // arm the block's barrier for the next step: its data can only be sent after this
              // step's MMAs on the block have retired (p_empty), so the arming always comes first
              if (elected && b != c) mbar_expect_tx(p_in(b), HALF_BYTES);
              fence_proxy_async();
              tc_fence_after();
              if (step == s0 && kc == 0) {  // the previous unit's dX must be drained first
                ok = mbar_wait_warp<true>(dx_empty, upar ^ 1u, abort_flag);
                if (!ok) break;
                tc_fence_after();
              }
            }
            ok = mbar_wait_warp<true>(ring_full(SLOTS_A + stage), phase, abort_flag);
            if (!ok) break;
            tc_fence_after();
            // A = W^T: two 64-wide h boxes (4096 B apart), each G2_KV lines of 128 bytes.
            const uint64_t adesc =
                make_smem_desc(ring + (SLOTS_A + stage) * SLOT_BYTES, 4096, 1024);
            if (elected) {
              for (int hb = 0; hb < p.nhb; ++hb) {
                const uint32_t d = tmem_base + hb * 128;
                // 16 K rows (vocabulary) per MMA = 2048 bytes = +128 in >>4 units
                umma_f16_ss_pair(d, adesc + 512u * hb, bdesc, idesc2, acc0);
                umma_f16_ss_pair(d, adesc + 512u * hb + 128u, bdesc + 128u, idesc2, 1u);
              }
              umma_commit_pair_mask(ring_empty(SLOTS_A + stage), pair_mask);
              // block kc / 4 of every P buffer this pair reads is free once these MMAs retire:
              // tell the CTA that produces it (the other pair's commit completes its barrier)
              if ((kc & (KC_PER_BLOCK - 1)) == KC_PER_BLOCK - 1)
                umma_commit_pair_mask(p_empty, static_cast<uint16_t>(1u << (kc / KC_PER_BLOCK)));
            }
            acc0 = 1u;
            bdesc += 256u;  // next 32 vocabulary lines of P
            if (++stage == SLOTS_B) {
              stage = 0;
              phase ^= 1u;
            }
          }
          g2par ^= 1u;
        }
        if (ok && elected) umma_commit_pair_mask(dx_full, pair_mask);
        upar ^= 1u;
      }
      if (!ok && elected) {
        *abort_flag = 1;
        atomicCAS(p.status, DEV_OK, DEV_TIMEOUT_BWD_MMA);
      }
    } else {
      // Pair peer: no MMAs to issue. This warp arms the local P barrier each step and relays
      // its completion to the leader, whose MMAs read this CTA's P buffer as well.
      const bool elected = elect_one_sync();
      const uint32_t p_peer_leader0 = mapa_shared(p_peer(0), leader);
      uint32_t par = 0;
      bool ok = true;
      if (elected)
        for (uint32_t b = 0; b < CL; ++b)
          if (b != c) mbar_expect_tx(p_in(b), HALF_BYTES);
      for (long long u = u_first; u < u_last && ok; u = unit_next(u)) {
        int s0, s1;
        unit_steps(u, s0, s1);
        for (int s = s0; s < s1 && ok; ++s) {
          for (uint32_t b = 0; b < CL; ++b) {
            ok = mbar_wait_warp<true>(p_in(b), par, abort_flag);
            if (!ok) break;
            if (elected) {
              mbar_arrive_remote(p_peer_leader0 + 8u * b);
              if (b != c) mbar_expect_tx(p_in(b), HALF_BYTES);   // next step (see the leader)
            }
          }
          par ^= 1u;
        }
      }
      if (!ok && elected) {
        *abort_flag = 1;
        atomicCAS(p.status, DEV_OK, DEV_TIMEOUT_BWD_MMA);
      }
    }
  } else {
    // ------------------------------- epilogue warps (every CTA) -----------------------
    const int quad = warp & 3;
    const int vi = quad * 32 + lane;  // TMEM lane: vocabulary row in G1, h column in G2
    const int et = (warp - 4) * 32 + lane;  // 0..127: index among the epilogue threads
    const uint32_t lane_bits = static_cast<uint32_t>(quad * 32) << 16;
    uint32_t scount = 0, ucount = 0;
    bool ok = true;
    const uint32_t s_empty_leader = mapa_shared(s_empty, leader);
    const uint32_t dx_empty_leader = mapa_shared(dx_empty, leader);
    // Line of vocabulary row vi: 128 bytes, 16-byte chunks XOR-swizzled by (vi & 7); block c of a
    // P buffer starts at line c * 128, the staging area holds one block.
    const uint32_t own_block = p_base + c * HALF_BYTES;
    const uint32_t own_line = own_block + vi * 128;
    const uint32_t stage_line = stage_buf + vi * 128;
    const uint32_t p_xor = static_cast<uint32_t>(vi & 7);
    const bool copy_warp = (warp == 4);
    const bool copy_lane = copy_warp && elect_one_sync();
    for (long long u = u_first; u < u_last && ok; u = unit_next(u)) {
      const int rt = unit_rt(u);
      const bool direct = (u < full_len);
      const int hs0 = (unit_pass(u) * CL + static_cast<int>(c)) * hs;
      int s0, s1;
      unit_steps(u, s0, s1);
      // ---- per-row constants of this unit (thread et loads row et) -------------------
      float* row_c2 = row_data;                             // -lse*log2e + log2(scale)
      float* row_rs = row_c2 + BM;                          // cew / scale
      int* row_tg = reinterpret_cast<int*>(row_rs + BM);    // local target id or -1
      // every warp must be done reading the previous unit's constants (drain) first
      ok = mbar_wait_warp(rd_free, (ucount & 1u) ^ 1u, abort_flag);
      if (!ok) break;
      {
        const int row = rt * BM + et;
        float c2 = NEG_BIG, rs = 0.f;
        int tg = -1;
        if (row < p.n) {
          const float w = p.cew[row];
          if (w != 0.f) {
            // e^(z-lse) * p_scale == 2^(z*log2e - lse*log2e + log2(p_scale))
            c2 = -p.lse[row] * LOG2E + (p.p_scale == 1.f ? 0.f : 10.f);
            rs = w / p.p_scale;
            const long long t = p.target[row] - p.vocab_offset;
            // the onehot term belongs to the unit whose vocabulary range holds the target
            if (t >= static_cast<long long>(s0) * STEP_V &&
                t < min(static_cast<long long>(s1) * STEP_V, static_cast<long long>(p.v)))
              tg = static_cast<int>(t);
          }
        }
        row_c2[et] = c2;
        row_rs[et] = rs;
        row_tg[et] = tg;
      }
      mbar_arrive(rd_ready);
      ok = mbar_wait_warp(rd_ready, ucount & 1u, abort_flag);
      if (!ok) break;
      // Software-pipelined over the steps of the unit with two register sets: raw logits of
      // step s+1 (r0..r3) and packed P of step s (pk). After P(s) is packed, the two remaining
      // actions - hand P(s) to the consumers (needs their buffers free) and pull the logits of
      // step s+1 out of TMEM (needs G1(s+1) finished) - run in whichever order they become
      // possible, so the G1 stream is never held up by a G2 stream that lags, or vice versa.
      uint32_t r0[32], r1[32], r2[32], r3[32];
      uint32_t pk[64];
      auto drain_logits = [&]() {
        tc_fence_after();
        tmem_ld32(tmem_base + S_COL + lane_bits + 0, r0);
        tmem_ld32(tmem_base + S_COL + lane_bits + 32, r1);
        tmem_ld32(tmem_base + S_COL + lane_bits + 64, r2);
        tmem_ld32(tmem_base + S_COL + lane_bits + 96, r3);
        tmem_ld_wait();
        // one arrival per warp: __syncwarp orders the lanes' TMEM reads before the elected
        // lane's cluster-scope release
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive_remote(s_empty_leader);
      };
      auto exp_pack = [&](const uint32_t (&r)[32], int ch, bool v_ok) {
#pragma unroll
        for (int j = 0; j < 32; j += 4) {
          const float4 c2v = *reinterpret_cast<const float4*>(row_c2 + ch * 32 + j);
          float e0 = ex2_approx(fmaf(__uint_as_float(r[j + 0]), LOG2E, c2v.x));
          float e1 = ex2_approx(fmaf(__uint_as_float(r[j + 1]), LOG2E, c2v.y));
          float e2 = ex2_approx(fmaf(__uint_as_float(r[j + 2]), LOG2E, c2v.z));
          float e3 = ex2_approx(fmaf(__uint_as_float(r[j + 3]), LOG2E, c2v.w));
          if (!v_ok) e0 = e1 = e2 = e3 = 0.f;
          pk[ch * 16 + j / 2 + 0] = pack2<kFmt>(e0, e1);
          pk[ch * 16 + j / 2 + 1] = pack2<kFmt>(e2, e3);
        }
      };
      auto hand_over = [&]() -> bool {
        // rows 0..63 (pk[0..31]) are consumed by ranks 0 and 2, rows 64..127 by ranks 1 and 3:
        // the half this CTA consumes goes into its own P buffer, the other one is staged
#pragma unroll
        for (int hf = 0; hf < 2; ++hf) {
          const uint32_t line = (static_cast<uint32_t>(hf) == half) ? own_line : stage_line;
#pragma unroll
          for (int q = 0; q < 8; ++q) {
            const int o = hf * 32 + q * 4;
            st_shared_v4(line + ((static_cast<uint32_t>(q) ^ p_xor) << 4), pk[o], pk[o + 1],
                         pk[o + 2], pk[o + 3]);
          }
        }
        fence_proxy_async();  // the lines are read by the async proxy (bulk copies, MMAs)
        __syncwarp();
        if (lane == 0) {
          mbar_arrive(p_in(c));      // a quarter of the own block of the own buffer is in place
          mbar_arrive(stage_ready);
        }
        if (copy_warp) {
          if (!mbar_wait_warp(stage_ready, scount & 1u, abort_flag)) return false;
          if (copy_lane) {
            // own half -> the CTA of the other pair that consumes the same rows
            bulk_copy_to_cluster(mapa_shared(own_block, c ^ 2u), own_block, HALF_BYTES,
                                 mapa_shared(p_in(c), c ^ 2u));
            // staged half -> the two CTAs that consume the other rows
            bulk_copy_to_cluster(mapa_shared(own_block, c ^ 1u), stage_buf, HALF_BYTES,
                                 mapa_shared(p_in(c), c ^ 1u));
            bulk_copy_to_cluster(mapa_shared(own_block, c ^ 3u), stage_buf, HALF_BYTES,
                                 mapa_shared(p_in(c), c ^ 3u));
          }
        }
        return true;
      };
      ok = mbar_wait_warp<true>(s_full, scount & 1u, abort_flag);
      if (!ok) break;
      drain_logits();
      for (int s = s0; s < s1 && ok; ++s, ++scount) {
        const bool v_ok = (s * STEP_V + static_cast<int>(c) * BV + vi) < p.v;
        exp_pack(r0, 0, v_ok);
        exp_pack(r1, 1, v_ok);
        exp_pack(r2, 2, v_ok);
        exp_pack(r3, 3, v_ok);
        bool stored = false, drained = (s + 1 >= s1);
        const long long t0 = clock64();
        while (ok && !(stored && drained)) {
          // every consumer must be done with the previous contents of its P buffer
          if (!stored &&
              __all_sync(0xffffffffu, mbar_test_wait_cluster(p_empty, (scount & 1u) ^ 1u))) {
            ok = hand_over();
            stored = true;
          }
          if (ok && !drained &&
              __all_sync(0xffffffffu, mbar_test_wait_cluster(s_full, (scount + 1u) & 1u))) {
            drain_logits();
            drained = true;
          }
          if (__any_sync(0xffffffffu, *abort_flag != 0 || clock64() - t0 > WAIT_LIMIT_CYCLES))
            ok = false;
        }
      }
      if (!ok) break;
      // ---- drain this CTA's dHidden^T slice: lane = h column, TMEM column = token row ----
      ok = mbar_wait_warp<true>(dx_full, ucount & 1u, abort_flag);
      if (!ok) break;
      tc_fence_after();
      // direct: dx[row, hcol]; partial: piece buffer [piece][left-over tile][128][pass width]
      const int pass_w = CL * hs;
      const int pcol0 = static_cast<int>(c) * hs;   // first column of this CTA inside the pass
      float* out;
      size_t out_ld;
      if (direct) {
        out = p.dx + static_cast<size_t>(rt) * BM * p.h + (hs0 - pcol0);
        out_ld = static_cast<size_t>(p.h);
      } else {
        out = p.dx_part + (static_cast<size_t>(cluster_id / p.rem_tp) * p.rem_tp +
                           cluster_id % p.rem_tp) * BM * pass_w;
        out_ld = static_cast<size_t>(pass_w);
      }
      for (int hb = 0; hb < p.nhb; ++hb) {
        const int hcol = hs0 + hb * 128 + vi;
        const int ocol = pcol0 + hb * 128 + vi;
#pragma unroll 1
        for (int ch = 0; ch < 4; ++ch) {
          uint32_t r[32];
          tmem_ld32(tmem_base + lane_bits + hb * 128 + ch * 32, r);
          tmem_ld_wait();
          if (hcol < p.h) {
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              const int rr = ch * 32 + j;
              const int row = rt * BM + rr;
              if (row < p.n) {
                const float rs = row_rs[rr];
                float val = __uint_as_float(r[j]) * rs;
                const int tg = row_tg[rr];
                if (tg >= 0)  // -cew * W[target, h]   (rs * p_scale == cew)
                  val -= rs * p.p_scale * load16<kFmt>(p.w, static_cast<size_t>(tg) * p.h + hcol);
                out[static_cast<size_t>(rr) * out_ld + ocol] = val;
              }
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        mbar_arrive_remote(dx_empty_leader);
        mbar_arrive(rd_free);
      }
      ++ucount;
    }
    if (!ok && lane == 0) {
      *abort_flag = 1;
      atomicCAS(p.status, DEV_OK, DEV_TIMEOUT_BWD_EPILOGUE);
    }
  }

  tc_fence_before();
  __syncthreads();
  cluster_arrive();  // nobody leaves while a peer may still store into, or arrive on, this CTA
  cluster_wait();
  tc_fence_after();
  if (warp == 1) tmem_dealloc_pair(tmem_base, TMEM_COLS);
}

}  // namespace esep
