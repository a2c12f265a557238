// Single-sweep training kernel of the LM head: one pass over the vocabulary computes the logits
// tiles ONCE and produces both the softmax statistics (loss, entropy, argmax) and the raw dHidden
// accumulator, so a training step executes 4*H*V*N flops instead of the 6*H*V*N of the
// forward sweep + recomputing backward sweep. Logits never leave the SM.
//
// Replaces the reference's whole per-chunk sequence (solution/head/op.py:87-100):
//     torch.mm(x, W.t()) ; head_row_softmax_kernel pass 1 and pass 2 ; torch.mm(g, W) ; scale.
//
// The softmax weights are taken relative to a per-row reference m_ref that is fixed BEFORE the
// sweep (the row maximum over a vocabulary prefix, from the forward kernel on those rows of W):
//     p[v, r] = e^(z[v, r] - m_ref[r])            (any positive size: rounded to bf16 for the GEMM)
//     raw dX[r, :] = sum_v p[v, r] W[v, :]         s[r] = sum_v p      t[r] = sum_v p (z - m_ref)
// and the caller's row kernel finishes: lse = m_ref + ln s, entropy = ln s - t / s,
// dX = cew (raw / s - W[target]) (with the target's own term treated separately, see below). No
// rescaling of accumulators is ever needed. m_ref is the prefix
// maximum plus REF_MARGIN = 40: fp32 / bf16 then hold p for logits from 47 below the prefix
// maximum (e^-47 of the largest weight: nothing) to 115 above it; a row that goes beyond raises
// `overflow` and the host's guarded two-kernel path recomputes the call.
//
// Geometry, operand layouts, TMA rings, the two independent MMA streams (G1: S^T = W_block x^T,
// G2: dX^T += W^T P) and the P exchange between the four CTAs of a cluster are those of
// head_bwd_kernel (head_bwd.cuh). Differences:
//   * P is bf16 whatever the model's type; G2 reads its W operand through `tmap_w2`, which the
//     host points at a bf16 copy of W when the model is fp16 (tcgen05.mma kind::f16 takes A and B
//     of one format), G1 reads the model's own W;
//   * eight epilogue warps (thread = vocabulary row x one 64-row half of the tile) so that the
//     extra per-row reductions fit the register file: per 32-row chunk a butterfly over the warp
//     turns "each lane holds 32 rows of its own vocabulary row" into "each lane holds one row
//     summed over the warp's 32 vocabulary rows" in 31 shuffles; the row maximum comes from the
//     same butterfly with fmaxf on the exact fp32 logits, and only when some row of the chunk
//     beats its running maximum (strictly: an earlier, i.e. lower, vocabulary index keeps equal
//     values) a second pass finds the lowest lane that holds that maximum (kernels.py:60, 75:
//     first index of the max). Every exponential is computed once and feeds both the row sums
//     and the packed P;
//   * the accumulator is drained raw; the -onehot term and all scaling moved to the row kernel;
//   * the row's TARGET entry is left out of P and of the sums: for a confident row p_target / s is
//     1 - tiny, and forming it from a bf16-rounded p would lose the tiny part. The row kernel adds
//     the target's own term in fp32: with s_rest the sum over the other entries and
//     p_t = e^(z_target - m_ref),  dX = cew (raw / s - (s_rest / s) W[target]),  ce = log1p(s_rest / p_t).
#pragma once

#include "head_norm.cuh"

namespace esep {

enum : int {
  DEV_TIMEOUT_TRN_PRODUCER = 301,
  DEV_TIMEOUT_TRN_MMA = 302,
  DEV_TIMEOUT_TRN_EPILOGUE = 303,
};

struct TrainParams {
  int n, h, v;            // n: rows the arrays below are laid out for (and swept, unless n_dev)
  const int* n_dev;       // null, or device word: only rows [0, *n_dev) are swept (*n_dev <= n);
                          // the work split is then derived on the device (sweep_split)
  int nhb;                // 128-wide H blocks per CTA (1..3)
  int total_steps;        // ceil(ceil(v / 128) / 4)
  const float* m_ref;     // [n] row maximum over the vocabulary prefix (REF_MARGIN is added here)
  const long long* target;  // [n] target ids; a valid target's entry is excluded from P and the sums
  float* dx;              // [n, h] raw accumulator of the directly written tiles
  float* dx_part;         // [rem_splits, rem_tp * 128 rows, pass width] pieces of left-over tiles
  // Per-row partial statistics, 16 slots (4 CTAs x 4 lane quadrants) per vocabulary run, written by
  // pass 0 only. Direct tiles: st_*[slot][row]; left-over tiles: lo_*[run * 16 + slot][j * 128 + r].
  float* st_s;
  float* st_t;
  float* st_max;          // largest logit of the slot's vocabulary rows (-inf if none), exact
  int* st_idx;            // its vocabulary index: the lowest one among equal logits
  float* lo_s;
  float* lo_t;
  float* lo_max;
  int* lo_idx;
  int w2_is_3d;
  int* overflow;          // set to 1 when a row's maximum is more than OVERFLOW_NATS above m_ref
  int* status;
};

namespace trn {
using namespace bwd;
static constexpr int EPI_WARPS = 8;
static constexpr int THREADS_T = 128 + EPI_WARPS * 32;   // 384
static constexpr float REF_MARGIN = 40.f;      // added to the prefix maximum: the reference m_ref
static constexpr float OVERFLOW_NATS = 75.f;   // largest z - m_ref the sweep accepts
static constexpr int ROWDATA_T = 2 * BM * 4;             // c2[128], local target id [128]
// barriers: full[6] empty[6] s_full s_empty p_empty dx_full dx_empty rd_ready rd_free stage_ready
//           p_in[4] p_peer[4]
static constexpr int NUM_BARS_T = 2 * SLOTS + 8 + 2 * CL;
static constexpr int SMEM_BYTES_T =
    1024 + P_BYTES + STAGE_BYTES + SLOTS * SLOT_BYTES + NUM_BARS_T * 8 + 64 + 16 + ROWDATA_T;
static_assert(SMEM_BYTES_T <= 232448, "exceeds the 227 KiB of shared memory a CTA may use");
}  // namespace trn

// v[j] (j = 0..31) of every lane -> returns, in lane l, the sum over all lanes of their v[l].
// 31 shuffles; v is destroyed.
__device__ __forceinline__ float warp_transpose_sum(float (&v)[32], int lane) {
#pragma unroll
  for (int w = 16; w >= 1; w >>= 1) {
    const bool up = (lane & w) != 0;
#pragma unroll
    for (int k = 0; k < w; ++k) {
      const float send = up ? v[k] : v[k + w];
      const float keep = up ? v[k + w] : v[k];
      v[k] = keep + __shfl_xor_sync(0xffffffffu, send, w);
    }
  }
  return v[0];
}

template <int kFmt>
__global__ void __launch_bounds__(trn::THREADS_T, 1)
head_train_kernel(const __grid_constant__ CUtensorMap tmap_x,    // x [n, h], box {64 k, 64 rows}
                  const __grid_constant__ CUtensorMap tmap_w1,   // W [v, h], box {64 k, 128 v}
                  const __grid_constant__ CUtensorMap tmap_w2,   // bf16 W as {64 h, v, h/64}, box
                                                                 // {64, 32, 6} (or 2-D, {64 h, 32 v})
                  const TrainParams p) {
  using namespace trn;
  if (p.n_dev != nullptr && *p.n_dev <= 0) return;   // no rows on this path (same for every CTA)
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
  const int misc_off = P_BYTES + STAGE_BYTES + SLOTS * SLOT_BYTES + NUM_BARS_T * 8;
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(gen_base + misc_off);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(gen_base + misc_off + 8);
  float* row_c2 = reinterpret_cast<float*>(gen_base + ((misc_off + 64 + 15) & ~15));  // float4 reads
  int* row_tg = reinterpret_cast<int*>(row_c2 + BM);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t c = cluster_ctarank();
  const uint32_t leader = c & ~1u;
  const bool is_leader = (c == leader);
  const uint32_t half = c & 1u;             // which 64 token rows this CTA feeds as B operand
  const uint16_t pair_mask = static_cast<uint16_t>(3u << leader);
  const int cluster_id = blockIdx.x / CL;
  const int kblocks = (p.h + BK - 1) / BK;
  // Work decomposition: the one of head_bwd_kernel (full rounds in lock step, then one
  // vocabulary run per cluster for the left-over tiles).
  const int n_clusters = gridDim.x / CL;
  const int hs = p.nhb * 128;
  const int n_rows = p.n_dev != nullptr ? min(*p.n_dev, p.n) : p.n;   // rows swept by this launch
  const int n_row_tiles = (n_rows + BM - 1) / BM;
  const int n_passes = (p.h + CL * hs - 1) / (CL * hs);
  const SweepSplit split =
      sweep_split(static_cast<long long>(n_row_tiles) * n_passes, n_clusters, p.total_steps);
  const long long full_len = static_cast<long long>(split.full_rounds) * p.total_steps;
  const bool has_rem = cluster_id < split.rem_tp * split.rem_splits;
  const long long u_first = (full_len > 0 || has_rem) ? 0 : 1;
  const long long u_last = full_len + (has_rem ? 1 : 0);

  if (threadIdx.x == 0) {
    for (int s = 0; s < SLOTS; ++s) {
      mbar_init(ring_full(s), 1);
      mbar_init(ring_empty(s), 1);
    }
    mbar_init(s_full, 1);                   // pair commit
    mbar_init(s_empty, 2 * EPI_WARPS);      // epilogue warps of both CTAs (leader's barrier)
    for (uint32_t b = 0; b < CL; ++b) {
      // own block: the epilogue warps that write it; other blocks: the arming arrive (+ 16 KiB)
      mbar_init(p_in(b), b == c ? EPI_WARPS / 2 : 1);
      mbar_init(p_peer(b), 1);              // relay arrive from the pair peer
    }
    mbar_init(rd_free, EPI_WARPS);
    mbar_init(stage_ready, EPI_WARPS);      // every line of this step's P block is in place
    mbar_init(p_empty, 2);                  // one commit per pair, after THIS CTA's block is consumed
    mbar_init(dx_full, 1);
    mbar_init(dx_empty, 2 * EPI_WARPS);
    mbar_init(rd_ready, EPI_WARPS * 32);
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
  cluster_arrive();
  cluster_wait();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  auto unit_tp = [&](long long u) {
    return u < full_len ? static_cast<int>(u / p.total_steps) * n_clusters + cluster_id
                        : split.full_rounds * n_clusters + cluster_id % split.rem_tp;
  };
  auto unit_rt = [&](long long u) { return unit_tp(u) % n_row_tiles; };
  auto unit_pass = [&](long long u) { return unit_tp(u) / n_row_tiles; };
  auto unit_steps = [&](long long u, int& s0, int& s1) {
    if (u < full_len) {
      s0 = 0;
      s1 = p.total_steps;
    } else {
      s0 = (cluster_id / split.rem_tp) * split.steps_per_split;
      s1 = min(p.total_steps, s0 + split.steps_per_split);
    }
  };
  auto unit_next = [&](long long u) { return u < full_len ? u + p.total_steps : u + 1; };

  if (warp == 0) {
    // ------------------- G1 producer (every CTA; whole warp, one lane issues) -----------
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
      atomicCAS(p.status, DEV_OK, DEV_TIMEOUT_TRN_PRODUCER);
    }
  } else if (warp == 2) {
    // ------------------- G2 producer (every CTA; whole warp, one lane issues) -----------
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
              tma_load_3d_pair(sa, &tmap_w2, bar, 0, vrow, hs0 / 64);
            } else {
#pragma unroll
              for (int b = 0; b < 6; ++b)
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
      atomicCAS(p.status, DEV_OK, DEV_TIMEOUT_TRN_PRODUCER);
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
          ok = mbar_wait_warp<true>(s_empty, g1par ^ 1u, abort_flag);
          if (!ok) break;
          tc_fence_after();
          for (int kb = 0; kb < kblocks; ++kb) {
            ok = mbar_wait_warp<true>(ring_full(stage), phase, abort_flag);
            if (!ok) break;
            tc_fence_after();
            const uint32_t sa = ring + stage * SLOT_BYTES;
            const uint64_t adesc = make_smem_desc(sa, 16, 1024);
            const uint64_t bdesc = make_smem_desc(sa + 16384, 16, 1024);
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
        atomicCAS(p.status, DEV_OK, DEV_TIMEOUT_TRN_MMA);
      }
    }
  } else if (warp == 3) {
    if (is_leader) {
      // ----------------- G2 issuer (pair leader; whole warp, one lane issues) -----------
      const bool elected = elect_one_sync();
      constexpr uint32_t idesc2 = make_idesc(1, 256, BM, 1, 1);  // bf16, MN-major A and B
      uint32_t stage = 0, phase = 0, g2par = 0, upar = 0;
      bool ok = true;
      if (elected)   // first step: 16 KiB from each of the three other CTAs
        for (uint32_t b = 0; b < CL; ++b)
          if (b != c) mbar_expect_tx(p_in(b), HALF_BYTES);
      for (long long u = u_first; u < u_last && ok; u = unit_next(u)) {
        int s0, s1;
        unit_steps(u, s0, s1);
        for (int step = s0; step < s1 && ok; ++step) {
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
              if (step == s0 && kc == 0) {
                ok = mbar_wait_warp<true>(dx_empty, upar ^ 1u, abort_flag);
                if (!ok) break;
                tc_fence_after();
              }
            }
            ok = mbar_wait_warp<true>(ring_full(SLOTS_A + stage), phase, abort_flag);
            if (!ok) break;
            tc_fence_after();
            const uint64_t adesc =
                make_smem_desc(ring + (SLOTS_A + stage) * SLOT_BYTES, 4096, 1024);
            if (elected) {
              for (int hb = 0; hb < p.nhb; ++hb) {
                const uint32_t d = tmem_base + hb * 128;
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
            bdesc += 256u;
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
        atomicCAS(p.status, DEV_OK, DEV_TIMEOUT_TRN_MMA);
      }
    } else {
      // Pair peer: arms the local P barrier each step and relays its completion to the leader.
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
        atomicCAS(p.status, DEV_OK, DEV_TIMEOUT_TRN_MMA);
      }
    }
  } else {
    // ------------------------------- epilogue warps (every CTA) -----------------------
    const int quad = warp & 3;                  // TMEM lane quadrant of this warp
    const int hf = (warp - 4) >> 2;             // which 64 rows of the tile this warp handles
    const int vi = quad * 32 + lane;            // TMEM lane: vocabulary row in G1, h column in G2
    const int et = (warp - 4) * 32 + lane;      // 0..255: index among the epilogue threads
    const uint32_t lane_bits = static_cast<uint32_t>(quad * 32) << 16;
    const uint32_t s_cols = tmem_base + S_COL + lane_bits + hf * 64;
    uint32_t scount = 0, ucount = 0;
    bool ok = true;
    const uint32_t s_empty_leader = mapa_shared(s_empty, leader);
    const uint32_t dx_empty_leader = mapa_shared(dx_empty, leader);
    // One 128-byte line per (vocabulary row, 64-row half), 16-byte chunks XOR-swizzled by (vi & 7).
    // The half this CTA consumes goes into its own P buffer, the other one into the staging area.
    const uint32_t own_block = p_base + c * HALF_BYTES;
    const bool writes_own = (static_cast<uint32_t>(hf) == half);
    const uint32_t line = (writes_own ? own_block : stage_buf) + vi * 128;
    const uint32_t p_xor = static_cast<uint32_t>(vi & 7);
    const bool copy_warp = (warp == 4);
    const bool copy_lane = copy_warp && elect_one_sync();
    for (long long u = u_first; u < u_last && ok; u = unit_next(u)) {
      const int rt = unit_rt(u);
      const bool direct = (u < full_len);
      const int pass = unit_pass(u);
      const int hs0 = (pass * CL + static_cast<int>(c)) * hs;
      int s0, s1;
      unit_steps(u, s0, s1);
      // ---- per-row constant of this unit: c2[r] = -m_ref[r] * log2(e) --------------------
      ok = mbar_wait_warp(rd_free, (ucount & 1u) ^ 1u, abort_flag);
      if (!ok) break;
      if (et < BM) {
        const int row = rt * BM + et;
        float c2 = NEG_BIG;
        int tg = -1;
        if (row < n_rows) {
          c2 = -(p.m_ref[row] + REF_MARGIN) * LOG2E;
          const long long t = p.target[row];
          if (t >= 0 && t < p.v) tg = static_cast<int>(t);
        }
        row_c2[et] = c2;
        row_tg[et] = tg;
      }
      mbar_arrive(rd_ready);
      ok = mbar_wait_warp(rd_ready, ucount & 1u, abort_flag);
      if (!ok) break;
      // Running statistics: lane l owns rows hf*64 + ch*32 + l (ch = 0, 1) of the tile, summed
      // over the 32 vocabulary rows of this warp and over the steps of the unit.
      float s_run[2] = {0.f, 0.f}, t_run[2] = {0.f, 0.f};
      float m_run[2] = {-INFINITY, -INFINITY};
      int i_run[2] = {0, 0};
      uint32_t z0[32], z1[32];   // raw logits of the next step (two 32-row chunks)
      uint32_t pk[32];           // packed bf16 P of the current step (64 rows)
      auto drain_logits = [&]() {
        tc_fence_after();
        tmem_ld32(s_cols + 0, z0);
        tmem_ld32(s_cols + 32, z1);
        tmem_ld_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive_remote(s_empty_leader);
      };
      // p = e^(z - m_ref) of one 32-row chunk (0 for the target entry and past the vocabulary).
      auto exp4 = [&](const uint32_t (&z)[32], int j, const float* c2p, const int* tgp, int my_v,
                      bool v_ok, float (&a)[4], float (&e)[4]) {
        const float4 c2v = *reinterpret_cast<const float4*>(c2p + j);
        a[0] = fmaf(__uint_as_float(z[j + 0]), LOG2E, c2v.x);
        a[1] = fmaf(__uint_as_float(z[j + 1]), LOG2E, c2v.y);
        a[2] = fmaf(__uint_as_float(z[j + 2]), LOG2E, c2v.z);
        a[3] = fmaf(__uint_as_float(z[j + 3]), LOG2E, c2v.w);
        const int4 tg4 = *reinterpret_cast<const int4*>(tgp + j);   // the target entry stays out
        e[0] = (!v_ok || tg4.x == my_v) ? 0.f : ex2_approx(a[0]);
        e[1] = (!v_ok || tg4.y == my_v) ? 0.f : ex2_approx(a[1]);
        e[2] = (!v_ok || tg4.z == my_v) ? 0.f : ex2_approx(a[2]);
        e[3] = (!v_ok || tg4.w == my_v) ? 0.f : ex2_approx(a[3]);
      };
      // The packed bf16 P alone (passes over the hidden dimension that do not own the statistics).
      auto chunk_pack = [&](const uint32_t (&z)[32], int ch, bool v_ok, int vbase) {
        const float* c2p = row_c2 + hf * 64 + ch * 32;
        const int* tgp = row_tg + hf * 64 + ch * 32;
        const int my_v = vbase + lane;
#pragma unroll
        for (int j = 0; j < 32; j += 4) {
          float a[4], e[4];
          exp4(z, j, c2p, tgp, my_v, v_ok, a, e);
          pk[ch * 16 + j / 2 + 0] = pack2<1>(e[0], e[1]);
          pk[ch * 16 + j / 2 + 1] = pack2<1>(e[2], e[3]);
        }
      };
      // Row maxima, the row sums s = sum p, t = sum p (z - m_ref), and the packed P. Destroys z.
      auto chunk_stats = [&](uint32_t (&z)[32], int ch, bool v_ok, int vbase) {
        const float* c2p = row_c2 + hf * 64 + ch * 32;
        const int* tgp = row_tg + hf * 64 + ch * 32;
        const int my_v = vbase + lane;
        float tmp[32];
        // Largest logit per row over this warp's 32 vocabulary rows: the butterfly leaves, in lane
        // l, the exact maximum of row l. Which vocabulary row holds it is looked up only when a
        // row beats its running maximum (rare once the sweep is under way).
#pragma unroll
        for (int j = 0; j < 32; ++j) tmp[j] = v_ok ? __uint_as_float(z[j]) : -INFINITY;
#pragma unroll
        for (int w = 16; w >= 1; w >>= 1) {
          const bool up = (lane & w) != 0;
#pragma unroll
          for (int k = 0; k < w; ++k) {
            const float send = up ? tmp[k] : tmp[k + w];
            const float keep = up ? tmp[k + w] : tmp[k];
            tmp[k] = fmaxf(keep, __shfl_xor_sync(0xffffffffu, send, w));
          }
        }
        {
          const float cm = tmp[0];
          // strict: an equal value met earlier sits at a lower vocabulary index and stays
          const bool better = cm > m_run[ch];
          if (__any_sync(0xffffffffu, better)) {
            int first = 0;
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              const float mj = __shfl_sync(0xffffffffu, cm, j);
              const unsigned hit =
                  __ballot_sync(0xffffffffu, v_ok && __uint_as_float(z[j]) == mj);
              if (lane == j) first = __ffs(hit) - 1;   // lowest lane = lowest vocabulary row
            }
            if (better) {
              m_run[ch] = cm;
              i_run[ch] = vbase + first;
            }
          }
        }
#pragma unroll
        for (int j = 0; j < 32; j += 4) {
          float a[4], e[4];
          exp4(z, j, c2p, tgp, my_v, v_ok, a, e);
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            tmp[j + i] = e[i];
            // q = p * (z - m_ref) in nats; the logits registers are free now
            z[j + i] = __float_as_uint(e[i] * (a[i] * LN2));
          }
          pk[ch * 16 + j / 2 + 0] = pack2<1>(e[0], e[1]);
          pk[ch * 16 + j / 2 + 1] = pack2<1>(e[2], e[3]);
        }
        s_run[ch] += warp_transpose_sum(tmp, lane);
#pragma unroll
        for (int j = 0; j < 32; ++j) tmp[j] = __uint_as_float(z[j]);
        t_run[ch] += warp_transpose_sum(tmp, lane);
      };
      auto hand_over = [&]() -> bool {
#pragma unroll
        for (int q = 0; q < 8; ++q)
          st_shared_v4(line + ((static_cast<uint32_t>(q) ^ p_xor) << 4), pk[q * 4 + 0],
                       pk[q * 4 + 1], pk[q * 4 + 2], pk[q * 4 + 3]);
        fence_proxy_async();  // the lines are read by the async proxy (bulk copies, MMAs)
        __syncwarp();
        if (lane == 0) {
          if (writes_own) mbar_arrive(p_in(c));   // a quarter of the own block of the own buffer
          mbar_arrive(stage_ready);
        }
        if (copy_warp) {
          if (!mbar_wait_warp(stage_ready, scount & 1u, abort_flag)) return false;
          if (copy_lane) {
            bulk_copy_to_cluster(mapa_shared(own_block, c ^ 2u), own_block, HALF_BYTES,
                                 mapa_shared(p_in(c), c ^ 2u));
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
        const int vbase = s * STEP_V + static_cast<int>(c) * BV + quad * 32;
        const bool v_ok = (vbase + lane) < p.v;
        bool stored = false, drained = (s + 1 >= s1);
        // One exponential per logit: in the pass that owns the statistics the same values feed the
        // row sums and the packed P. P of this step is not needed before the G2 stream has worked
        // through the previous step's blocks, so forming the sums first costs it nothing.
        if (pass == 0) {
          chunk_stats(z0, 0, v_ok, vbase);
          chunk_stats(z1, 1, v_ok, vbase);
        } else {
          chunk_pack(z0, 0, v_ok, vbase);
          chunk_pack(z1, 1, v_ok, vbase);
        }
        const long long t0 = clock64();
        while (ok && !(stored && drained)) {
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
      // ---- drain this CTA's raw dHidden^T slice: lane = h column, TMEM column = token row ----
      ok = mbar_wait_warp<true>(dx_full, ucount & 1u, abort_flag);
      if (!ok) break;
      tc_fence_after();
      const int pass_w = CL * hs;
      const int pcol0 = static_cast<int>(c) * hs;
      float* out;
      size_t out_ld;
      if (direct) {
        out = p.dx + static_cast<size_t>(rt) * BM * p.h + (hs0 - pcol0);
        out_ld = static_cast<size_t>(p.h);
      } else {
        out = p.dx_part + (static_cast<size_t>(cluster_id / split.rem_tp) * split.rem_tp +
                           cluster_id % split.rem_tp) * BM * pass_w;
        out_ld = static_cast<size_t>(pass_w);
      }
      for (int hb = 0; hb < p.nhb; ++hb) {
        const int hcol = hs0 + hb * 128 + vi;
        const int ocol = pcol0 + hb * 128 + vi;
#pragma unroll 1
        for (int ch = 0; ch < 2; ++ch) {
          uint32_t r[32];
          tmem_ld32(tmem_base + lane_bits + hb * 128 + hf * 64 + ch * 32, r);
          tmem_ld_wait();
          if (hcol < p.h) {
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              const int rr = hf * 64 + ch * 32 + j;
              if (rt * BM + rr < n_rows)
                out[static_cast<size_t>(rr) * out_ld + ocol] = __uint_as_float(r[j]);
            }
          }
        }
      }
      // ---- statistics of this unit (the first pass over the hidden dimension owns them) -------
      if (pass == 0) {
        const int slot = static_cast<int>(c) * 4 + quad;
#pragma unroll
        for (int ch = 0; ch < 2; ++ch) {
          const int rr = hf * 64 + ch * 32 + lane;
          const int row = rt * BM + rr;
          if (row < n_rows) {
            size_t o;
            float *ds, *dt, *dm;
            int* di;
            if (direct) {
              o = static_cast<size_t>(slot) * p.n + row;
              ds = p.st_s; dt = p.st_t; dm = p.st_max; di = p.st_idx;
            } else {
              const int run = cluster_id / split.rem_tp, j = cluster_id % split.rem_tp;
              o = (static_cast<size_t>(run) * 16 + slot) *
                      (static_cast<size_t>(split.rem_tp) * BM) +
                  static_cast<size_t>(j) * BM + rr;
              ds = p.lo_s; dt = p.lo_t; dm = p.lo_max; di = p.lo_idx;
            }
            ds[o] = s_run[ch];
            dt[o] = t_run[ch];
            dm[o] = m_run[ch];
            di[o] = i_run[ch];
            // -inf (no vocabulary row in range) and NaN compare false
            if (fmaf(m_run[ch], LOG2E, row_c2[rr]) > OVERFLOW_NATS * LOG2E)
              atomicExch(p.overflow, 1);
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
      atomicCAS(p.status, DEV_OK, DEV_TIMEOUT_TRN_EPILOGUE);
    }
  }

  tc_fence_before();
  __syncthreads();
  cluster_arrive();
  cluster_wait();
  tc_fence_after();
  if (warp == 1) tmem_dealloc_pair(tmem_base, TMEM_COLS);
}


}  // namespace esep
