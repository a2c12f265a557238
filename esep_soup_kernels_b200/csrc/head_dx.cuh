// dHidden from stored logits: the second half of the two-sweep training path.
//
// With 180 GB of HBM the logits of a batch can stay in memory for a few milliseconds (fp16,
// 1.3 GB for 4 340 rows x 151 936): the forward sweep (head_fwd_kernel<.., kStore>) writes
// logit - m_ref as fp16 once, and this kernel turns them into softmax weights on the fly and
// multiplies by W. Against the fused single pass (head_train.cuh) this computes every logit once
// AND lets each GEMM run in its best shape: here a CTA pair owns TWO 128-row tiles, so a W tile
// that enters shared memory is used for 256 rows (the single pass: 128, which is what bounds it),
// and the clusters are pairs, which every SM of the GPU can host.
// Replaces the reference's `torch.mm(g, W)` over the live rows (solution/head/op.py:99-100) and
// pass 2 of its row kernel (solution/head/kernels.py:84-93: g = softmax - onehot).
//
//   D^T[h, row] += W^T[h, v] * P[v, row],   P = e^(z - lse) (x 1024 for fp16), target entry = 0
//
// A operand: W [v, h] as MN-major tiles through the 3-D tensor map (64 h, 32 v, 4) - 256 hidden
// columns per CTA, two accumulator blocks of 128 lanes x 256 columns (all 512 TMEM columns).
// B operand: the stored logits [row, vocab] are K-major as they are. Sixteen warps read them from
// global memory two steps ahead (registers), turn them into weights with one packed 2^x per two
// entries and store the tile to shared memory in the 128-byte-swizzled layout the MMA expects.
// They do not pass through shared memory as logits: what bounds these kernels is the 128 B/clk of
// shared-memory bandwidth per SM - the MMAs read 64 B/clk of operands at N = 256 (96 at N = 128,
// which is what holds the single pass at 0.6 of the tensor peak), the W tiles arrive at 32 B/clk,
// and the P tiles are written at 16.
//
// Work: unit = (pair of row tiles, 512-column slice of H); a unit's vocabulary is cut into
// `segs` runs when there are too few units to fill the pairs (dx_split). Runs are handed out
// segment-major, so at any time all pairs work within two neighbouring vocabulary segments and
// share their W tiles through L2. Every run writes its partial D^T as a piece [256 rows, 512
// columns] fp32; the row-finish kernel adds a row's pieces in a fixed order.
// Warps (736 threads): 0 = TMA producer of the W tiles, 1 = MMA issuer (pair leader) + TMEM owner;
// of warps 2..22 the sixteen that do NOT share the MMA issuer's scheduler (warp % 4 != 1) transform,
// so that the one thread that feeds the tensor pipe never queues behind them; warps 5, 9, 13, 17
// only help with the drain of the accumulators at the end of a run (TMEM lanes 32..63 can only be
// read by warps with warp % 4 == 1); warp 5 also relays "tile ready" from the transform warps'
// shared-memory counter to the leader's mbarrier. Every wait is bounded.
//
// kDirect (the default form of the path): the forward sweep has stored the weights themselves,
// bf16 2^((z - m_ref - 40) log2 e) with the target's entry zero, so P needs no transform: warp 18
// (which drains nothing) brings each step's tile in with two TMA boxes of 64 weights x 128 rows
// per CTA, the layout above, and the sixteen warps only drain. The row's factor
// 2^((m_ref + 40 - lse) log2 e) is applied by the row finish. Measured at 4 340 x 1536 x 151 936:
// tensor pipe busy 92 % of the launch (72 % with the transform), 1.25 against 1.67 ms.
#pragma once

#include <algorithm>

#include "head_bwd.cuh"
#include "head_fwd.cuh"

namespace esep {

enum : int {
  DEV_TIMEOUT_DX_PRODUCER = 401,
  DEV_TIMEOUT_DX_MMA = 402,
  DEV_TIMEOUT_DX_TRANSFORM = 403,
};

namespace dxk {
static constexpr int ROWS = 256;          // token rows per unit (two tiles, one per CTA)
static constexpr int SLICE = 512;         // hidden columns per unit (256 per CTA)
static constexpr int BLK_V = 128;         // vocabulary entries per step
static constexpr int KV = 32;             // vocabulary rows per W slot
static constexpr int P_SLOT = 128 * BLK_V * 2;      // 32 KiB: this CTA's rows x one step
static constexpr int P_SLOTS = 4;
static constexpr int W_SLOT = KV * 256 * 2;         // 16 KiB
static constexpr int W_SLOTS = 6;
static constexpr int T_WARPS = 16;                  // transform warps
static constexpr int THREADS = 23 * 32;              // 736: see the warp roles
static constexpr int NUM_BARS = 2 * W_SLOTS + 2 * P_SLOTS + 4;
static constexpr int SMEM_BYTES =
    1024 + P_SLOTS * P_SLOT + W_SLOTS * W_SLOT + NUM_BARS * 8 + 64 + 128 * 8;
static constexpr float FP16_SCALE_LOG2 = 10.f;      // P x 1024 (the reference's G_SCALE)
static constexpr float DIRECT_OVERFLOW_NATS = 75.f; // largest z - m_ref whose weight bf16 is trusted with
}  // namespace dxk

// How the units of a launch are cut and handed out; the same on the host (buffer sizes), in the
// kernel and in the row finish.
struct DxSplit {
  int row_pairs, slices, units, steps, segs, seg_steps, runs;
};
__host__ __device__ inline DxSplit dx_split(int n_rows, int h, int v, int n_pairs) {
  DxSplit r;
  r.row_pairs = (n_rows + dxk::ROWS - 1) / dxk::ROWS;
  r.slices = (h + dxk::SLICE - 1) / dxk::SLICE;
  r.units = r.row_pairs * r.slices;
  r.steps = (v + dxk::BLK_V - 1) / dxk::BLK_V;
  r.segs = 1;
  if (n_pairs < 1) n_pairs = 1;
  if (r.units > 0 && r.units < 8 * n_pairs) {
    int kmax = 8 * n_pairs / r.units;
    if (kmax > 16) kmax = 16;
    if (kmax > r.steps) kmax = r.steps;
    float best = -1.f;
    for (int k = 1; k <= kmax; ++k) {
      const int waves = (r.units * k + n_pairs - 1) / n_pairs;
      const float eff = static_cast<float>(r.units * k) / (static_cast<float>(waves) * n_pairs);
      if (eff > best + 1e-6f) {
        best = eff;
        r.segs = k;
      }
      if (eff >= 0.97f) break;
    }
  }
  r.seg_steps = r.steps > 0 ? (r.steps + r.segs - 1) / r.segs : 0;
  r.segs = r.seg_steps > 0 ? (r.steps + r.seg_steps - 1) / r.seg_steps : 0;
  r.runs = r.units * r.segs;
  return r;
}
// Upper bound of dx_split(n', ...).runs over all n' <= n_rows (pieces the buffer must hold).
__host__ inline long long dx_max_runs(int n_rows, int h, int v, int n_pairs) {
  const DxSplit full = dx_split(n_rows, h, v, n_pairs);   // units grow with the rows; segs <= 16
  const long long cut = std::min<long long>(8LL * n_pairs, 16LL * full.units);
  return std::max<long long>(full.units, cut);
}

struct DxParams {
  int n, h, v;               // n: rows the arrays hold; the launch sweeps rows [0, *n_dev)
  const int* n_dev;
  const __half* z;           // [n][zpitch] stored (logit - m_ref) log2 e
  long long zpitch;
  const float* kexp;         // [n] integer part of (m_ref - lse) * log2(e), + 10: P = 2^(d + kexp),
                             //     d = the stored fp16 value; the fraction is applied by the
                             //     row finish in fp32 (head_dx_rowconst_kernel)
  const long long* target;   // [n] compact targets; the entry of a valid target is left out of P
  float* pieces;             // [runs][256][512] fp32
  int* status;
};

// kDirect: the buffer already holds the softmax weights as bf16 (the forward sweep's second store
// mode); a producer warp brings their tiles in by TMA, in the layout the MMAs read, and no warp
// transforms anything. W is then a bf16 tensor whatever the model's type (kFmt = 1).
template <int kFmt, bool kDirect = false>   // type of W and of P: 0 = fp16, 1 = bf16
__global__ void __launch_bounds__(dxk::THREADS, 1)
head_dx_kernel(const __grid_constant__ CUtensorMap tmap_w,   // W as {64 h, v, h/64}, box {64, 32, 4}
               const __grid_constant__ CUtensorMap tmap_z,   // kDirect: weights [n, zpitch], box {64, 128}
               const DxParams p) {
  using namespace dxk;
  if (min(*p.n_dev, p.n) <= 0) return;   // no rows on this path (every CTA reads the same count)
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* gen_base = smem_raw + (base - raw);
  const uint32_t p_base = base;
  const uint32_t w_base = base + P_SLOTS * P_SLOT;
  const uint32_t bars = w_base + W_SLOTS * W_SLOT;
  auto w_full = [&](uint32_t s) { return bars + 8u * s; };
  auto w_empty = [&](uint32_t s) { return bars + 8u * (W_SLOTS + s); };
  auto p_ready = [&](uint32_t s) { return bars + 8u * (2 * W_SLOTS + s); };
  auto p_empty = [&](uint32_t s) { return bars + 8u * (2 * W_SLOTS + P_SLOTS + s); };
  const uint32_t dx_full = bars + 8u * (2 * W_SLOTS + 2 * P_SLOTS);
  const uint32_t dx_empty = dx_full + 8u;
  const uint32_t rc_ready = dx_full + 16u;    // the row constants of a run are in shared memory
  const uint32_t rc_free = dx_full + 24u;     // ... and no transform warp reads them any more
  const int misc_off = P_SLOTS * P_SLOT + W_SLOTS * W_SLOT + NUM_BARS * 8;
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(gen_base + misc_off);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(gen_base + misc_off + 8);
  // p_cnt[s]: transform warps that have finished slot s, counted up for ever (plain shared-memory
  // atomics: see the relay warp below)
  int* p_cnt = reinterpret_cast<int*>(gen_base + misc_off + 16);
  float* row_c2 = reinterpret_cast<float*>(gen_base + misc_off + 64);
  int* row_tg = reinterpret_cast<int*>(row_c2 + 128);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t c = cluster_ctarank();
  const bool is_leader = (c == 0);
  const int pair_id = blockIdx.x >> 1;
  const int n_pairs = gridDim.x >> 1;
  const int n_rows = min(*p.n_dev, p.n);
  const DxSplit sp = dx_split(n_rows, p.h, p.v, n_pairs);

  if (threadIdx.x == 0) {
    for (uint32_t s = 0; s < W_SLOTS; ++s) {
      mbar_init(w_full(s), 1);
      mbar_init(w_empty(s), 1);
    }
    for (uint32_t s = 0; s < P_SLOTS; ++s) {
      // the relay warps of both CTAs, or the leader's expect-tx for both CTAs' tiles
      mbar_init(p_ready(s), kDirect ? 1 : 2);
      p_cnt[s] = 0;
      mbar_init(p_empty(s), 1);
    }
    mbar_init(dx_full, 1);
    mbar_init(dx_empty, 2 * T_WARPS);
    mbar_init(rc_ready, T_WARPS * 32);
    mbar_init(rc_free, T_WARPS);
    *abort_flag = 0;
    fence_barrier_init();
    fence_proxy_async();
    tma_prefetch_desc(&tmap_w);
    if (kDirect) tma_prefetch_desc(&tmap_z);
  }
  if (warp == 1) {
    tmem_alloc_pair(smem_u32(const_cast<uint32_t*>(tmem_slot)), 512);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  cluster_arrive();
  cluster_wait();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  // run w -> (segment, row pair, slice); slices vary fastest so that neighbouring pairs read the
  // same logits at the same time
  auto run_seg = [&](int w) { return w / sp.units; };
  auto run_rp = [&](int w) { return (w % sp.units) / sp.slices; };
  auto run_q = [&](int w) { return (w % sp.units) % sp.slices; };
  auto run_steps = [&](int w, int& s0, int& s1) {
    s0 = run_seg(w) * sp.seg_steps;
    s1 = min(sp.steps, s0 + sp.seg_steps);
  };

  if (warp == 0) {
    // ------------------- TMA producer of W (both CTAs; whole warp, one lane issues) -----
    const bool elected = elect_one_sync();
    uint32_t ws = 0, wph = 0;
    bool ok = true;
    const uint32_t w_full_leader0 = mapa_shared(w_full(0), 0);
    for (int w = pair_id; w < sp.runs && ok; w += n_pairs) {
      const int hblk = (run_q(w) * SLICE + static_cast<int>(c) * 256) / 64;
      int s0, s1;
      run_steps(w, s0, s1);
      for (int st = s0; st < s1 && ok; ++st) {
        for (int kc = 0; kc < BLK_V / KV; ++kc) {
          ok = mbar_wait_warp<true>(w_empty(ws), wph ^ 1u, abort_flag);
          if (!ok) break;
          if (elected) {
            if (is_leader) mbar_expect_tx(w_full(ws), 2 * W_SLOT);
            tma_load_3d_pair(w_base + ws * W_SLOT, &tmap_w, w_full_leader0 + 8u * ws, 0,
                             st * BLK_V + kc * KV, hblk);
          }
          if (++ws == W_SLOTS) {
            ws = 0;
            wph ^= 1u;
          }
        }
      }
    }
    if (!ok && elected) {
      *abort_flag = 1;
      atomicCAS(p.status, DEV_OK, DEV_TIMEOUT_DX_PRODUCER);
    }
  } else if (warp == 1) {
    // ------------------- MMA issuer (pair leader; whole warp, one lane issues) ----------
    if (is_leader) {
      const bool elected = elect_one_sync();
      constexpr uint32_t idesc = make_idesc(kFmt, 256, 256, 1, 0);   // A MN-major, B K-major
      constexpr uint16_t kPairMask = 3;
      uint32_t ws = 0, wph = 0, ps = 0, pph = 0, upar = 0;
      bool ok = true;
      for (int w = pair_id; w < sp.runs && ok; w += n_pairs) {
        int s0, s1;
        run_steps(w, s0, s1);
        ok = mbar_wait_warp<true>(dx_empty, upar ^ 1u, abort_flag);   // accumulators drained
        if (!ok) break;
        tc_fence_after();
        uint32_t acc = 0;
        for (int st = s0; st < s1 && ok; ++st) {
          ok = mbar_wait_warp<true>(p_ready(ps), pph, abort_flag);
          if (!ok) break;
          tc_fence_after();
          for (int kc = 0; kc < BLK_V / KV; ++kc) {
            ok = mbar_wait_warp<true>(w_full(ws), wph, abort_flag);
            if (!ok) break;
            tc_fence_after();
            const uint64_t adesc = make_smem_desc(w_base + ws * W_SLOT, 4096, 1024);
            // 32 vocabulary entries = 64 bytes inside the 128-byte line of a 64-entry sub-tile
            const uint64_t bdesc =
                make_smem_desc(p_base + ps * P_SLOT + (kc >> 1) * (P_SLOT / 2), 16, 1024) +
                4u * (kc & 1);
            if (elected) {
#pragma unroll
              for (int hb = 0; hb < 2; ++hb) {
                const uint32_t d = tmem_base + hb * 256;
                umma_f16_ss_pair(d, adesc + 512u * hb, bdesc, idesc, acc);
                umma_f16_ss_pair(d, adesc + 512u * hb + 128u, bdesc + 2u, idesc, 1u);
              }
              umma_commit_pair_mask(w_empty(ws), kPairMask);
              if (kc == BLK_V / KV - 1) umma_commit_pair_mask(p_empty(ps), kPairMask);
            }
            acc = 1u;
            if (++ws == W_SLOTS) {
              ws = 0;
              wph ^= 1u;
            }
          }
          if (++ps == P_SLOTS) {
            ps = 0;
            pph ^= 1u;
          }
        }
        if (ok && elected) umma_commit_pair_mask(dx_full, kPairMask);
        upar ^= 1u;
      }
      if (!ok && elected) {
        *abort_flag = 1;
        atomicCAS(p.status, DEV_OK, DEV_TIMEOUT_DX_MMA);
      }
    }
  } else if (kDirect && warp == 18) {
    // ------------------- TMA producer of P (both CTAs; this warp drains nothing) ----------
    const bool elected = elect_one_sync();
    uint32_t ps = 0, pph = 0;
    bool ok = true;
    const uint32_t p_ready_leader0 = mapa_shared(p_ready(0), 0);
    for (int w = pair_id; w < sp.runs && ok; w += n_pairs) {
      const int row0 = run_rp(w) * ROWS + static_cast<int>(c) * 128;
      int s0, s1;
      run_steps(w, s0, s1);
      for (int st = s0; st < s1 && ok; ++st) {
        ok = mbar_wait_warp<true>(p_empty(ps), pph ^ 1u, abort_flag);
        if (!ok) break;
        if (elected) {
          if (is_leader) mbar_expect_tx(p_ready(ps), 2 * P_SLOT);
          const uint32_t dst = p_base + ps * P_SLOT;
          tma_load_2d_pair(dst, &tmap_z, p_ready_leader0 + 8u * ps, st * BLK_V, row0);
          tma_load_2d_pair(dst + P_SLOT / 2, &tmap_z, p_ready_leader0 + 8u * ps, st * BLK_V + 64,
                           row0);
        }
        if (++ps == P_SLOTS) {
          ps = 0;
          pph ^= 1u;
        }
      }
    }
    if (!ok && elected) {
      *abort_flag = 1;
      atomicCAS(p.status, DEV_OK, DEV_TIMEOUT_DX_PRODUCER);
    }
  } else {
    // ------------------- transform warps: logits -> P; drain at the end of a run ----------
    const int quad = warp & 3;                  // TMEM lane quadrant this warp may read
    const bool does_transform = !kDirect && quad != 1;
    const int tt = ((warp - 2) - ((warp - 1) >> 2)) * 32 + lane;   // 0..511 among the transformers
    // which 128 of the 512 accumulator columns this warp drains (four warps per quadrant do)
    const int part = quad < 2 ? (warp >> 2) - 1 : (warp >> 2);
    const bool does_drain = part >= 0 && part < 4;
    const uint32_t lane_bits = static_cast<uint32_t>(quad * 32) << 16;
    const uint32_t p_ready_leader0 = mapa_shared(p_ready(0), 0);
    const uint32_t dx_empty_leader = mapa_shared(dx_empty, 0);
    // A slot holds two sub-tiles of 64 vocabulary entries; a sub-tile is 128 lines (rows) of
    // 128 bytes, 16-byte groups XOR-swizzled by (line & 7). Thread tt works on the rows tt >> 3
    // and 64 + (tt >> 3) of both sub-tiles, always on the logical group tt & 7 (8 entries).
    const int line_lo = tt >> 3;
    const int grp = tt & 7;
    const uint32_t phys = static_cast<uint32_t>(line_lo * 128 + ((grp ^ (line_lo & 7)) * 16));
    uint32_t ps = 0, pph = 0, upar = 0;
    long long relay_n = 0;      // steps this CTA's relay warp has passed on (slot use count)
    bool ok = true;
    for (int w = pair_id; w < sp.runs && ok; w += n_pairs) {
      const int row0 = run_rp(w) * ROWS + static_cast<int>(c) * 128;
      int s0, s1;
      run_steps(w, s0, s1);
      if (!kDirect && warp == 5) {
        // ---- relay: when all sixteen transform warps have finished a slot, tell the leader.
        // This warp has no loads in flight, so its arrive does not wait for any.
        for (int st = s0; st < s1 && ok; ++st) {
          const int want = T_WARPS * static_cast<int>(relay_n / P_SLOTS + 1);
          int have = 0;
          if (lane == 0) {
            const long long t0 = clock64();
            while ((have = *reinterpret_cast<volatile int*>(p_cnt + ps)) < want) {
              if (*abort_flag != 0 || clock64() - t0 > WAIT_LIMIT_CYCLES) break;
            }
          }
          have = __shfl_sync(0xffffffffu, have, 0);
          ok = have >= want;
          if (!ok) break;
          __syncwarp();
          if (lane == 0) mbar_arrive_remote(p_ready_leader0 + 8u * ps);
          ++relay_n;
          if (++ps == P_SLOTS) ps = 0;
        }
        if (!ok) break;
      }
      if (does_transform) {
      // per-row constants of this CTA's 128 rows (once the previous run's transforms are done)
      ok = mbar_wait_warp(rc_free, upar ^ 1u, abort_flag);
      if (!ok) break;
      if (tt < 128) {
        const int row = row0 + tt;
        float c2 = -60000.f;     // rows past the end: P = 0
        int tg = -1;
        if (row < n_rows) {
          c2 = p.kexp[row];
          const long long t = p.target[row];
          if (t >= 0 && t < p.v) tg = static_cast<int>(t);
        }
        row_c2[tt] = c2;
        row_tg[tt] = tg;
      }
      mbar_arrive(rc_ready);
      ok = mbar_wait_warp(rc_ready, upar, abort_flag);
      if (!ok) break;
      const __half2 k2r[2] = {__float2half2_rn(row_c2[line_lo]),
                              __float2half2_rn(row_c2[64 + line_lo])};
      const int tgr[2] = {row_tg[line_lo] - grp * 8, row_tg[64 + line_lo] - grp * 8};
      __syncwarp();
      if (lane == 0) mbar_arrive(rc_free);      // the constants are in registers now
      // this thread's two rows in the stored logits (null past the end of the buffer)
      const __half* zr[2];
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        const int row = row0 + r * 64 + line_lo;
        zr[r] = row < p.n ? p.z + static_cast<size_t>(row) * p.zpitch + grp * 8 : nullptr;
      }
      // in[.][it]: it & 1 = row, it >> 1 = sub-tile
      auto fetch = [&](int st, uint4 (&buf)[4]) {
#pragma unroll
        for (int it = 0; it < 4; ++it) {
          const __half* src = zr[it & 1];
          buf[it] = (src != nullptr && st < s1)
                        ? __ldg(reinterpret_cast<const uint4*>(src + st * BLK_V + (it >> 1) * 64))
                        : make_uint4(0u, 0u, 0u, 0u);
        }
      };
      auto emit = [&](int st, const uint4 (&buf)[4]) -> bool {
        if (!mbar_wait_warp(p_empty(ps), pph ^ 1u, abort_flag)) return false;
        const uint32_t slot = p_base + ps * P_SLOT + phys;
#pragma unroll
        for (int it = 0; it < 4; ++it) {
          const uint32_t in[4] = {buf[it].x, buf[it].y, buf[it].z, buf[it].w};
          uint32_t out[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            // two entries per instruction: P = 2^(d + k) <= 2^10.5 in fp16
            const __half2 arg = __hadd2(*reinterpret_cast<const __half2*>(&in[e]), k2r[it & 1]);
            const uint32_t pe = ex2_approx_f16x2(*reinterpret_cast<const uint32_t*>(&arg));
            if (kFmt == 0) {
              out[e] = pe;
            } else {
              // fp16 -> bf16 of two positive values with integer operations (the conversion
              // instructions share the XU pipe with the 2^x and would triple its load): round the
              // 10-bit mantissa to 7 bits (to nearest, ties to even), move the exponent (bias 15 -> 127), and keep zero for
              // what fp16 holds as zero or subnormal (below 2^-14 of a scale of 2^10).
              const uint32_t rne = pe + 0x00030003u + ((pe >> 3) & 0x00010001u);   // ties to even
              const uint32_t r = ((rne >> 3) & 0x1FFF1FFFu) + 0x38003800u;
              const uint32_t keep = ((pe & 0x0000FC00u) ? 0x0000FFFFu : 0u) |
                                    ((pe & 0xFC000000u) ? 0xFFFF0000u : 0u);
              out[e] = r & keep;
            }
          }
          // the target's entry (once per row and run): 0..7 when it sits in this group
          const unsigned tl = static_cast<unsigned>(tgr[it & 1] - (st * BLK_V + (it >> 1) * 64));
          if (tl < 8u) {
#pragma unroll
            for (int e = 0; e < 4; ++e)
              if (static_cast<unsigned>(e) == (tl >> 1)) out[e] &= (tl & 1u) ? 0x0000ffffu : 0xffff0000u;
          }
          st_shared_v4(slot + static_cast<uint32_t>((it >> 1) * (P_SLOT / 2) + (it & 1) * (64 * 128)),
                       out[0], out[1], out[2], out[3]);
        }
        fence_proxy_async_shared();   // the MMAs read the tile through the async proxy
        __syncwarp();
        // Not an mbarrier arrive: its release would wait for this warp's prefetched loads of the
        // next steps (measured: 1 600 of the 4 000 cycles a step took). The tile itself is already
        // ordered for the MMAs by the proxy fence above.
        if (lane == 0) atomicAdd(p_cnt + ps, 1);
        if (++ps == P_SLOTS) {
          ps = 0;
          pph ^= 1u;
        }
        return true;
      };
      uint4 buf_a[4], buf_b[4];   // logits of the next two steps, in flight while this one is turned
      fetch(s0, buf_a);
      fetch(s0 + 1, buf_b);
      for (int st = s0; st < s1 && ok; st += 2) {
        ok = emit(st, buf_a);
        fetch(st + 2, buf_a);
        if (ok && st + 1 < s1) ok = emit(st + 1, buf_b);
        fetch(st + 3, buf_b);
      }
      }
      if (!ok) break;
      // ---- drain D^T of this run: lane = hidden column, TMEM column = token row -------------
      if (does_drain) {
      ok = mbar_wait_warp<true>(dx_full, upar, abort_flag);
      if (!ok) break;
      tc_fence_after();
      float* piece = p.pieces + static_cast<size_t>(w) * ROWS * SLICE;
      {
        const int hb = part >> 1, chalf = part & 1;
        const int col = static_cast<int>(c) * 256 + hb * 128 + quad * 32 + lane;
#pragma unroll 1
        for (int ch = 0; ch < 4; ++ch) {
          uint32_t r[32];
          tmem_ld32(tmem_base + lane_bits + hb * 256 + chalf * 128 + ch * 32, r);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 32; ++j)
            piece[static_cast<size_t>(chalf * 128 + ch * 32 + j) * SLICE + col] =
                __uint_as_float(r[j]);
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_remote(dx_empty_leader);
      }
      upar ^= 1u;
    }
    if (!ok && lane == 0) {
      *abort_flag = 1;
      atomicCAS(p.status, DEV_OK, DEV_TIMEOUT_DX_TRANSFORM);
    }
  }

  tc_fence_before();
  __syncthreads();
  cluster_arrive();
  cluster_wait();
  tc_fence_after();
  if (warp == 1) tmem_dealloc_pair(tmem_base, 512);
}

// The per-row constants of the softmax weights for the swept rows, from the forward sweep's
// partial records (target entry left out of the sums; merge rule kernels.py:70-81):
// e^(z - lse) = 2^(d + c), d = the stored (z - m_ref) log2 e, c = (m_ref - lse) log2 e <= 0.
// kexp = round(c) + 10 goes into the exponent in fp16 (P <= 2^10.5; the + 10 keeps small weights
// out of fp16's subnormal range, as the reference's G_SCALE does, op.py:39), rscale =
// 2^(c - round(c) - 10) multiplies the finished sums in fp32.
__global__ void __launch_bounds__(128)
head_dx_rowconst_kernel(int n_cap, const int* __restrict__ n_dev, int n_vtiles, int fwd_pairs,
                        int part_cap, const float* __restrict__ pm, const float* __restrict__ ps,
                        const float* __restrict__ ptz, const long long* __restrict__ target, int v,
                        const float* __restrict__ m_ref, float* __restrict__ kexp,
                        float* __restrict__ rscale, int direct, int* __restrict__ overflow) {
  const int n_rows = min(*n_dev, n_cap);
  const int row = blockIdx.x * 128 + threadIdx.x;
  if (row >= n_rows) return;
  const FwdSplit fs = fwd_split_rows(n_rows, n_vtiles, fwd_pairs, part_cap);
  float m = NEG_BIG;
  for (int k = 0; k < fs.n_splits; ++k) m = fmaxf(m, pm[static_cast<size_t>(k) * fs.stride + row]);
  float s = 0.f, tz = 0.f;
  for (int k = 0; k < fs.n_splits; ++k) {
    const size_t o = static_cast<size_t>(k) * fs.stride + row;
    s += ps[o] * __expf(pm[o] - m);
    tz += ptz[o];
  }
  const long long t = target[row];
  if (t >= 0 && t < v) s += __expf(tz - m);
  const float lse = m + logf(s);
  if (direct) {
    const float ref = m_ref[row] + fwd::STORED_WEIGHT_MARGIN;
    const float c = fmaxf((ref - lse) * LOG2E, -30000.f);
    // The buffer holds 2^d as bf16: the whole factor is applied by the row finish. A row whose
    // largest logit is so far above m_ref that bf16 may not hold its weights sends the call to the
    // guarded second attempt, as in the single pass.
    kexp[row] = 0.f;
    rscale[row] = exp2f(c);
    if (!(m - ref <= dxk::DIRECT_OVERFLOW_NATS)) *overflow = 1;
    return;
  }
  const float c = fmaxf((m_ref[row] - lse) * LOG2E, -30000.f);
  const float ki = rintf(c);
  kexp[row] = ki + dxk::FP16_SCALE_LOG2;
  rscale[row] = exp2f(c - ki - dxk::FP16_SCALE_LOG2);
}

}  // namespace esep
