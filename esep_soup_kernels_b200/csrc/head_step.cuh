// Kernels around the two sweeps for a whole head step whose row classes are only known on the
// device: which rows are selected at all, which carry a loss term (they need dHidden and go
// through the training sweep) and which only need statistics (forward sweep). Nothing here
// synchronises with the host: counts stay in device memory and the sweeps read them there.
//
// Replaces the torch glue of the reference around its chunk loop:
//   solution/head/op.py:104-128     masks, live-first stable permutation (with its host sync),
//                                   un-permutation, loss = (cew * ce).sum()
//   solution/head/patch.py:443-487  label shift, row selection by attention mask, row gather and
//                                   cast, scatter of per-row CE / entropy back to [B, T], counts
#pragma once

#include "head_dx.cuh"
#include "head_train.cuh"

namespace esep {

// Device words shared by the kernels of one step (int[4] at `counts`):
//   [0] n_sweep  compact rows [0, n_sweep) go through the training sweep
//   [1] n_sel    compact rows [n_sweep, n_sel) go through the forward sweep only
//   [2] n_live   rows with a loss term and a non-zero weight
//   [3] unused
// CNT_SWEEP / CNT_SEL: the compact rows [0, n_sweep) need a gradient, [n_sweep, n_sel) statistics
// only. CNT_TRAIN: rows the single-pass kernels sweep, {CNT_ZERO, CNT_STORE}: the row range
// {0, rows} of the logits-storing sweep - one of the two is n_sweep, the other 0 (CNT_STORED says
// which path the call takes).
enum : int { CNT_SWEEP = 0, CNT_SEL = 1, CNT_LIVE = 2, CNT_TRAIN = 3, CNT_ZERO = 4, CNT_STORE = 5,
             CNT_STORED = 6 };

// Scalars written by head_step_scalars_kernel.
enum : int {
  MET_LOSS = 0,       // sum cew * ce
  MET_VALID = 1,      // rows whose target id lies in [0, v)
  MET_CORRECT = 2,    // of those, rows with argmax == target
  MET_ENT_VALID = 3,  // sum of entropy over those rows
  MET_LABELLED = 4,   // rows whose target is not -100 (the reference's `labelled`, patch.py:485)
  MET_ATTENDED = 5,   // attended rows (attention mask != 0; every row without a mask)
  MET_ENT_ATT = 6,    // sum of entropy over the attended rows (patch.py:600-606)
  MET_LIVE = 7,       // rows that took part in the gradient
  MET_COUNT = 8
};

struct StepPrepParams {
  int m, v, seq_len, need_grad;
  const long long* target;   // flat mode: [m] target ids (labels == null)
  const float* ce_weight;    // flat mode: [m] weights, or null for weight 1
  const long long* labels;   // step mode: [m] = [batch, seq_len] labels, target = label of t + 1
  const long long* attn;     // step mode: [m] attention mask or null (all rows selected)
  long long* tgt_o;          // [m] targets in the caller's row order
  long long* tgt_c;          // [m] targets in compact order (-1 past n_sel)
  float* cew_c;              // [m] masked weights in compact order (0 past n_sel)
  int* perm;                 // [m] compact -> caller row (-1 past n_sel)
  int* inv;                  // [m] caller row -> compact (-1: not selected)
  int* counts;
  int* overflow;             // cleared here
  int* status;               // cleared here
  int stored;                // training path of the rows with a gradient: 1 = two sweeps
};

// Target, weight and selection of caller row r (op.py:105-107; patch.py:446-458).
__device__ __forceinline__ void step_classify(const StepPrepParams& q, int r, long long& tg,
                                              float& w, bool& sel) {
  if (q.labels != nullptr) {
    const int t = r % q.seq_len;
    tg = (t + 1 < q.seq_len) ? q.labels[r + 1] : -100;   // pad right with -100, shift by one
    const bool has = tg != -100;
    sel = has || q.attn == nullptr || q.attn[r] != 0;
    w = has ? 1.f : 0.f;
  } else {
    tg = q.target[r];
    w = q.ce_weight != nullptr ? q.ce_weight[r] : 1.f;
    sel = true;
  }
  if (tg < 0 || tg >= q.v) w = 0.f;
}

// One block of 1024 threads: stable partition of the selected rows into "sweep" rows (loss term
// with non-zero weight, when a gradient is wanted) followed by the other selected rows.
// If at most one selected row in eight is of the second kind, they all go through the sweep
// (a separate forward launch for a handful of rows costs more than their share of the sweep).
__global__ void __launch_bounds__(1024) head_step_prep_kernel(const StepPrepParams q) {
  __shared__ int wa[32], wb[32], tot[2];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int chunk = (q.m + 1023) / 1024;
  const int r0 = min(q.m, tid * chunk), r1 = min(q.m, r0 + chunk);
  int a = 0, b = 0;
  for (int r = r0; r < r1; ++r) {
    long long tg;
    float w;
    bool sel;
    step_classify(q, r, tg, w, sel);
    if (sel) {
      if (q.need_grad && w != 0.f) ++a; else ++b;
    }
  }
  int ia = a, ib = b;   // inclusive scans over the warp
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int ta = __shfl_up_sync(0xffffffffu, ia, o), tb = __shfl_up_sync(0xffffffffu, ib, o);
    if (lane >= o) {
      ia += ta;
      ib += tb;
    }
  }
  if (lane == 31) {
    wa[warp] = ia;
    wb[warp] = ib;
  }
  __syncthreads();
  if (warp == 0) {
    int va = wa[lane], vb = wb[lane];
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int ta = __shfl_up_sync(0xffffffffu, va, o), tb = __shfl_up_sync(0xffffffffu, vb, o);
      if (lane >= o) {
        va += ta;
        vb += tb;
      }
    }
    wa[lane] = va;   // inclusive over warps
    wb[lane] = vb;
    if (lane == 31) {
      tot[0] = va;
      tot[1] = vb;
    }
  }
  __syncthreads();
  const int n_first = tot[0], n_other = tot[1], n_sel = n_first + n_other;
  int pa = (warp > 0 ? wa[warp - 1] : 0) + ia - a;            // exclusive prefix, first class
  int pb = n_first + (warp > 0 ? wb[warp - 1] : 0) + ib - b;  // second class follows the first
  for (int r = r0; r < r1; ++r) {
    long long tg;
    float w;
    bool sel;
    step_classify(q, r, tg, w, sel);
    q.tgt_o[r] = tg;
    int pos = -1;
    if (sel) {
      pos = (q.need_grad && w != 0.f) ? pa++ : pb++;
      q.perm[pos] = r;
      q.tgt_c[pos] = (tg >= 0 && tg < q.v) ? tg : -1;
      q.cew_c[pos] = w;
    }
    q.inv[r] = pos;
  }
  for (int pos = n_sel + tid; pos < q.m; pos += 1024) {
    q.perm[pos] = -1;
    q.tgt_c[pos] = -1;
    q.cew_c[pos] = 0.f;
  }
  if (tid == 0) {
    int n_sweep = 0;
    if (q.need_grad) n_sweep = (n_other * 8 <= n_sel) ? n_sel : n_first;
    q.counts[CNT_SWEEP] = n_sweep;
    q.counts[CNT_SEL] = n_sel;
    q.counts[CNT_LIVE] = n_first;
    const int stored = q.stored;
    q.counts[CNT_TRAIN] = stored ? 0 : n_sweep;
    q.counts[CNT_ZERO] = 0;
    q.counts[CNT_STORE] = stored ? n_sweep : 0;
    q.counts[CNT_STORED] = stored;
    *q.overflow = 0;
    *q.status = 0;
  }
}

// Compact copy of the selected rows in 16 bit: xc[pos, :] = x[perm[pos], :] (zeros past n_sel).
// x is 16-bit (kFmt) or fp32 (cast here: op.py:109). One block per compact row, 16-byte vectors.
template <int kFmt, bool kF32>
__global__ void __launch_bounds__(128)
head_step_gather_kernel(const void* __restrict__ x, const int* __restrict__ perm, int h,
                        void* __restrict__ xc) {
  const int pos = blockIdx.x;
  const int src = perm[pos];
  uint4* dst = reinterpret_cast<uint4*>(static_cast<uint8_t*>(xc) + static_cast<size_t>(pos) * h * 2);
  for (int c = threadIdx.x; c < h / 8; c += blockDim.x) {
    uint4 val = make_uint4(0u, 0u, 0u, 0u);
    if (src >= 0) {
      if (kF32) {
        const float4* s4 = reinterpret_cast<const float4*>(
            static_cast<const float*>(x) + static_cast<size_t>(src) * h) + 2 * c;
        const float4 lo = s4[0], hi = s4[1];
        val = make_uint4(pack2<kFmt>(lo.x, lo.y), pack2<kFmt>(lo.z, lo.w), pack2<kFmt>(hi.x, hi.y),
                         pack2<kFmt>(hi.z, hi.w));
      } else {
        val = reinterpret_cast<const uint4*>(static_cast<const uint8_t*>(x) +
                                             static_cast<size_t>(src) * h * 2)[c];
      }
    }
    dst[c] = val;
  }
}

// Finishes one row of the caller's batch (one block of 128 threads per row):
//   not selected                outputs 0, dHidden row 0
//   sweep row                   merges the sweep's partial statistics (sums add, the largest
//                               logit wins, lowest index among equals), adds the target's own term
//                               in fp32 and turns the raw accumulator of its compact row into
//                               dHidden (exact zeros when the weight is 0); or, when the sweep
//                               overflowed, takes what the guarded two-kernel pass left
//   forward-only row            merges the forward sweep's partial records (kernels.py:70-81)
// and writes everything at the caller's row index.
struct StepRowsParams {
  int m, h, v;
  int n_clusters, nhb, total_steps;       // geometry of the training sweep launch
  int n_vtiles, fwd_pairs, part_cap;      // geometry of the forward launch over the other rows
  const int* counts;
  const int* overflow;
  const int* inv;
  const void* xc;
  const void* w;
  const long long* tgt_c;
  const float* cew_c;
  const float* m_ref;
  const float *st_s, *st_t, *st_max, *lo_s, *lo_t, *lo_max;
  const int *st_idx, *lo_idx;
  const float* dx_part;
  const float* dxc;                       // [m, h] raw accumulators (or final rows after overflow)
  const float *pm, *ps, *pt, *ptz;        // forward partial records [split][row - n_sweep]
  const int* pidx;
  const float *f_lse, *f_tl, *f_ce, *f_ent, *f_cew;   // compact outputs of the guarded pass
  const float* f_max;                     // its merged record, field 0: the row maximum
  const long long* f_amax;
  float *lse, *tlogit, *ce, *ent, *cew_out;
  long long* amax;
  float* top;                             // null, or [m]: the largest logit of every selected row
  float* dx;                              // [m, h] or null (no gradient wanted)
  // Two-sweep training path (stored logits, head_dx.cuh): the swept rows' statistics come from
  // the storing forward sweep's partial records (target entry left out of the sums) and their
  // raw dHidden from the pieces of head_dx_kernel.
  int stored;                             // 0: single pass; 1: two sweeps
  int dx_pairs;                           // CTA pairs of the head_dx_kernel launch
  const float* g_rscale;                  // [m] what the summed pieces of a row are multiplied by
  const float *g_pm, *g_ps, *g_pt, *g_ptz;
  const int* g_pidx;
  const float* pieces;
};

// Merge of a row's partial records over the vocabulary runs of a forward sweep (kernels.py:70-81):
// block of 128 threads, thread k reads run k. Returns the maximum, and through the references the
// sums relative to it, the target logit and the lowest index of the maximum.
__device__ __forceinline__ float merge_partial_records(const float* pm, const float* ps,
                                                       const float* pt, const float* ptz,
                                                       const int* pidx, size_t o0,
                                                       const FwdSplit& fs, float (*sh_f)[4],
                                                       int* sh_i, float& s, float& t, float& tz,
                                                       int& idx) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float mk = NEG_BIG, sk = 0.f, tk = 0.f, tzk = 0.f;
  int ik = 0x7fffffff;
  if (static_cast<int>(threadIdx.x) < fs.n_splits) {   // n_splits <= 128 = blockDim
    const size_t o = o0 + static_cast<size_t>(threadIdx.x) * fs.stride;
    mk = pm[o];
    sk = ps[o];
    tk = pt[o];
    tzk = ptz[o];
    ik = pidx[o];
  }
  float big = mk;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) big = fmaxf(big, __shfl_xor_sync(0xffffffffu, big, o));
  if (lane == 0) sh_f[0][warp] = big;
  __syncthreads();
  big = fmaxf(fmaxf(sh_f[0][0], sh_f[0][1]), fmaxf(sh_f[0][2], sh_f[0][3]));
  __syncthreads();
  const float dl = mk - big;
  const float sc = __expf(dl);
  s = sk * sc;
  t = sc * (tk + sk * dl);
  tz = tzk;
  idx = (mk == big) ? ik : 0x7fffffff;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    s += __shfl_xor_sync(0xffffffffu, s, o);
    t += __shfl_xor_sync(0xffffffffu, t, o);
    tz += __shfl_xor_sync(0xffffffffu, tz, o);
    idx = min(idx, __shfl_xor_sync(0xffffffffu, idx, o));
  }
  if (lane == 0) {
    sh_f[0][warp] = s;
    sh_f[1][warp] = t;
    sh_f[2][warp] = tz;
    sh_i[warp] = idx;
  }
  __syncthreads();
  s = sh_f[0][0] + sh_f[0][1] + sh_f[0][2] + sh_f[0][3];
  t = sh_f[1][0] + sh_f[1][1] + sh_f[1][2] + sh_f[1][3];
  tz = sh_f[2][0] + sh_f[2][1] + sh_f[2][2] + sh_f[2][3];
  idx = min(min(sh_i[0], sh_i[1]), min(sh_i[2], sh_i[3]));
  return big;
}

// 12 blocks per SM: the kernel waits for its loads (pieces, records), so resident warps count for
// more than the 130 bytes of spills the 40-register cap costs (uncapped: 80 registers, 6 blocks per
// SM, 125 us at 4 340 x 1536 with DRAM at 30 % of its bandwidth; capped, the whole step is 0.04 ms
// shorter).
template <int kFmt>
__global__ void __launch_bounds__(128, 12) head_step_rows_kernel(const StepRowsParams q) {
  __shared__ float sh_f[4][4];
  __shared__ int sh_i[4];
  const int r = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int pos = q.inv[r];
  const int n_sweep = q.counts[CNT_SWEEP];
  float* drow = q.dx != nullptr ? q.dx + static_cast<size_t>(r) * q.h : nullptr;
  float o_lse = 0.f, o_tl = 0.f, o_ce = 0.f, o_ent = 0.f, o_cw = 0.f, o_top = 0.f;
  long long o_am = 0;
  enum { DX_ZERO, DX_COPY, DX_FINISH } dx_mode = DX_ZERO;
  float inv_s = 0.f, coef = 0.f;          // DX_FINISH: dx = cw (raw * inv_s - coef * W[target])
  long long tg = -1;

  if (pos >= 0 && pos < n_sweep && *q.overflow != 0) {
    o_lse = q.f_lse[pos];
    o_tl = q.f_tl[pos];
    o_ce = q.f_ce[pos];
    o_ent = q.f_ent[pos];
    o_cw = q.f_cew[pos];
    o_am = q.f_amax[pos];
    o_top = q.f_max[pos];
    dx_mode = DX_COPY;
  } else if (pos >= 0 && pos < n_sweep && q.stored != 0) {
    // ---- two-sweep path: records of the storing forward sweep + pieces of head_dx_kernel ------
    const FwdSplit fs = fwd_split_rows(n_sweep, q.n_vtiles, q.fwd_pairs, q.part_cap);
    float s_rest, t, tz;
    int idx;
    const float big = merge_partial_records(q.g_pm, q.g_ps, q.g_pt, q.g_ptz, q.g_pidx,
                                            static_cast<size_t>(pos), fs, sh_f, sh_i, s_rest, t,
                                            tz, idx);
    tg = q.tgt_c[pos];
    const bool valid = tg >= 0;
    float s = s_rest, p_t = 0.f;
    if (valid) {   // the target's own term, left out of the sums by the sweep
      p_t = __expf(tz - big);
      s += p_t;
      t += p_t * (tz - big);
    }
    const float log_s = logf(s);
    o_lse = big + log_s;
    o_ent = log_s - t / s;
    o_am = idx;
    o_top = big;
    o_tl = valid ? tz : 0.f;
    o_ce = valid ? (s_rest < p_t ? log1pf(s_rest / p_t) : (o_lse - tz)) : 0.f;
    o_cw = q.cew_c[pos];
    // dHidden = cew (sum_{v != t} p_v W_v - (1 - p_t) W_t), 1 - p_t = s_rest / s; the pieces hold
    // the first sum up to the row's factor g_rscale (p is already divided by s)
    coef = s_rest / s;
    dx_mode = o_cw != 0.f ? DX_FINISH : DX_ZERO;
    if (drow != nullptr && dx_mode == DX_FINISH) {
      const DxSplit ds = dx_split(n_sweep, q.h, q.v, q.dx_pairs);
      const int rp = pos / dxk::ROWS, rr = pos % dxk::ROWS;
      const size_t piece = static_cast<size_t>(dxk::ROWS) * dxk::SLICE;
      const float rs = q.g_rscale[pos];
      for (int c = threadIdx.x * 4; c < q.h; c += 128 * 4) {
        const int u = rp * ds.slices + c / dxk::SLICE;
        const float* src = q.pieces + static_cast<size_t>(u) * piece +
                           static_cast<size_t>(rr) * dxk::SLICE + (c % dxk::SLICE);
        float4 rawv = *reinterpret_cast<const float4*>(src);
        for (int k = 1; k < ds.segs; ++k) {
          const float4 b = *reinterpret_cast<const float4*>(src + static_cast<size_t>(k) * ds.units * piece);
          rawv.x += b.x;
          rawv.y += b.y;
          rawv.z += b.z;
          rawv.w += b.w;
        }
        const float4 wt = load4_16<kFmt>(q.w, (static_cast<size_t>(tg) * q.h + c) / 4);
        *reinterpret_cast<float4*>(drow + c) = make_float4(
            o_cw * (rawv.x * rs - coef * wt.x), o_cw * (rawv.y * rs - coef * wt.y),
            o_cw * (rawv.z * rs - coef * wt.z), o_cw * (rawv.w * rs - coef * wt.w));
      }
    }
  } else if (pos >= 0 && pos < n_sweep) {
    // ---- sweep row: partial statistics, all relative to m_ref ---------------------------------
    const int n_row_tiles = (n_sweep + 127) / 128;
    const int hs = q.nhb * 128;
    const int n_passes = (q.h + 4 * hs - 1) / (4 * hs);
    const SweepSplit sp =
        sweep_split(static_cast<long long>(n_row_tiles) * n_passes, q.n_clusters, q.total_steps);
    const int first_tp = sp.full_rounds * q.n_clusters;
    const int rt = pos / 128, rr = pos % 128;
    float s = 0.f, t = 0.f, mx = -INFINITY;
    int idx = 0x7fffffff;
    {
      const bool lo = rt >= first_tp;   // pass 0 of this row tile was swept in vocabulary runs
      const int nslots = lo ? sp.rem_splits * 16 : 16;
      const size_t stride = lo ? static_cast<size_t>(sp.rem_tp) * 128 : static_cast<size_t>(q.m);
      const size_t o0 =
          lo ? static_cast<size_t>(rt - first_tp) * 128 + rr : static_cast<size_t>(pos);
      const float* ps = lo ? q.lo_s : q.st_s;
      const float* pt = lo ? q.lo_t : q.st_t;
      const float* pm = lo ? q.lo_max : q.st_max;
      const int* pi = lo ? q.lo_idx : q.st_idx;
      for (int k = threadIdx.x; k < nslots; k += 128) {
        const size_t o = o0 + k * stride;
        s += ps[o];
        t += pt[o];
        const float mk = pm[o];
        const int ik = pi[o];
        if (mk > mx || (mk == mx && ik < idx)) {
          mx = mk;
          idx = ik;
        }
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      s += __shfl_xor_sync(0xffffffffu, s, o);
      t += __shfl_xor_sync(0xffffffffu, t, o);
      const float mk = __shfl_xor_sync(0xffffffffu, mx, o);
      const int ik = __shfl_xor_sync(0xffffffffu, idx, o);
      if (mk > mx || (mk == mx && ik < idx)) {
        mx = mk;
        idx = ik;
      }
    }
    // target logit: xc[pos, :] . W[target, :]
    tg = q.tgt_c[pos];
    const bool valid = tg >= 0;
    float tz = 0.f;
    if (valid)
      for (int c = threadIdx.x * 8; c < q.h; c += 128 * 8) {
        const float4 xa = load4_16<kFmt>(q.xc, (static_cast<size_t>(pos) * q.h + c) / 4);
        const float4 xb = load4_16<kFmt>(q.xc, (static_cast<size_t>(pos) * q.h + c) / 4 + 1);
        const float4 wa = load4_16<kFmt>(q.w, (static_cast<size_t>(tg) * q.h + c) / 4);
        const float4 wb = load4_16<kFmt>(q.w, (static_cast<size_t>(tg) * q.h + c) / 4 + 1);
        tz = fmaf(xa.x, wa.x, tz);
        tz = fmaf(xa.y, wa.y, tz);
        tz = fmaf(xa.z, wa.z, tz);
        tz = fmaf(xa.w, wa.w, tz);
        tz = fmaf(xb.x, wb.x, tz);
        tz = fmaf(xb.y, wb.y, tz);
        tz = fmaf(xb.z, wb.z, tz);
        tz = fmaf(xb.w, wb.w, tz);
      }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) tz += __shfl_xor_sync(0xffffffffu, tz, o);
    if (lane == 0) {
      sh_f[0][warp] = s;
      sh_f[1][warp] = t;
      sh_f[2][warp] = tz;
      sh_f[3][warp] = mx;
      sh_i[warp] = idx;
    }
    __syncthreads();
    s = sh_f[0][0] + sh_f[0][1] + sh_f[0][2] + sh_f[0][3];
    t = sh_f[1][0] + sh_f[1][1] + sh_f[1][2] + sh_f[1][3];
    tz = sh_f[2][0] + sh_f[2][1] + sh_f[2][2] + sh_f[2][3];
    mx = sh_f[3][0];
    idx = sh_i[0];
#pragma unroll
    for (int k = 1; k < 4; ++k)
      if (sh_f[3][k] > mx || (sh_f[3][k] == mx && sh_i[k] < idx)) {
        mx = sh_f[3][k];
        idx = sh_i[k];
      }
    // s, t so far leave out the target entry: add its own term in fp32
    const float m = q.m_ref[pos] + trn::REF_MARGIN;
    const float s_rest = s;
    float p_t = 0.f;
    if (valid) {
      p_t = __expf(tz - m);
      s += p_t;
      t += p_t * (tz - m);
    }
    const float log_s = logf(s);
    o_lse = m + log_s;
    o_ent = log_s - t / s;
    o_am = idx;
    o_top = mx;
    o_tl = valid ? tz : 0.f;
    // ln s - (z_t - m) = ln(1 + s_rest / p_t): the form without cancellation for confident rows
    o_ce = valid ? (s_rest < p_t ? log1pf(s_rest / p_t) : (o_lse - tz)) : 0.f;
    o_cw = q.cew_c[pos];
    // dHidden = cew (raw / s - (1 - p_t / s) W[target]),  1 - p_t / s = s_rest / s
    inv_s = 1.f / s;
    coef = s_rest * inv_s;
    dx_mode = o_cw != 0.f ? DX_FINISH : DX_ZERO;
    if (drow != nullptr && dx_mode == DX_FINISH) {
      const int pass_w = 4 * hs;
      for (int c = threadIdx.x * 4; c < q.h; c += 128 * 4) {   // pass widths are multiples of 512
        const int pass = c / pass_w;
        const int tp = pass * n_row_tiles + rt;
        float4 rawv;
        if (tp < first_tp) {
          rawv = *reinterpret_cast<const float4*>(q.dxc + static_cast<size_t>(pos) * q.h + c);
        } else {
          const size_t piece = static_cast<size_t>(sp.rem_tp) * 128 * pass_w;
          const float* src = q.dx_part +
                             (static_cast<size_t>(tp - first_tp) * 128 + rr) * pass_w +
                             (c - pass * pass_w);
          rawv = *reinterpret_cast<const float4*>(src);
          for (int k = 1; k < sp.rem_splits; ++k) {
            const float4 b = *reinterpret_cast<const float4*>(src + k * piece);
            rawv.x += b.x;
            rawv.y += b.y;
            rawv.z += b.z;
            rawv.w += b.w;
          }
        }
        const float4 wt = load4_16<kFmt>(q.w, (static_cast<size_t>(tg) * q.h + c) / 4);
        *reinterpret_cast<float4*>(drow + c) = make_float4(
            o_cw * (rawv.x * inv_s - coef * wt.x), o_cw * (rawv.y * inv_s - coef * wt.y),
            o_cw * (rawv.z * inv_s - coef * wt.z), o_cw * (rawv.w * inv_s - coef * wt.w));
      }
    }
  } else if (pos >= 0) {
    // ---- forward-only row: merge the partial records of its vocabulary runs --------------------
    const int n_sel = q.counts[CNT_SEL];
    const FwdSplit fs = fwd_split_rows(max(n_sel - n_sweep, 0), q.n_vtiles, q.fwd_pairs, q.part_cap);
    const size_t o0 = static_cast<size_t>(pos - n_sweep);
    float mk = NEG_BIG, sk = 0.f, tk = 0.f, tzk = 0.f;
    int ik = 0x7fffffff;
    if (static_cast<int>(threadIdx.x) < fs.n_splits) {   // n_splits <= 128 = blockDim
      const size_t o = o0 + static_cast<size_t>(threadIdx.x) * fs.stride;
      mk = q.pm[o];
      sk = q.ps[o];
      tk = q.pt[o];
      tzk = q.ptz[o];
      ik = q.pidx[o];
    }
    float big = mk;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) big = fmaxf(big, __shfl_xor_sync(0xffffffffu, big, o));
    if (lane == 0) sh_f[0][warp] = big;
    __syncthreads();
    big = fmaxf(fmaxf(sh_f[0][0], sh_f[0][1]), fmaxf(sh_f[0][2], sh_f[0][3]));
    __syncthreads();
    const float dl = mk - big;
    const float sc = __expf(dl);
    float s = sk * sc, t = sc * (tk + sk * dl), tz = tzk;
    int idx = (mk == big) ? ik : 0x7fffffff;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      s += __shfl_xor_sync(0xffffffffu, s, o);
      t += __shfl_xor_sync(0xffffffffu, t, o);
      tz += __shfl_xor_sync(0xffffffffu, tz, o);
      idx = min(idx, __shfl_xor_sync(0xffffffffu, idx, o));
    }
    if (lane == 0) {
      sh_f[0][warp] = s;
      sh_f[1][warp] = t;
      sh_f[2][warp] = tz;
      sh_i[warp] = idx;
    }
    __syncthreads();
    s = sh_f[0][0] + sh_f[0][1] + sh_f[0][2] + sh_f[0][3];
    t = sh_f[1][0] + sh_f[1][1] + sh_f[1][2] + sh_f[1][3];
    tz = sh_f[2][0] + sh_f[2][1] + sh_f[2][2] + sh_f[2][3];
    idx = min(min(sh_i[0], sh_i[1]), min(sh_i[2], sh_i[3]));
    const float log_s = logf(s);
    tg = q.tgt_c[pos];
    const bool valid = tg >= 0;
    o_lse = big + log_s;
    o_ent = log_s - t / s;
    o_am = idx;
    o_top = big;
    o_tl = valid ? tz : 0.f;
    o_ce = valid ? (o_lse - tz) : 0.f;
    o_cw = q.cew_c[pos];
  }

  if (threadIdx.x == 0) {
    q.lse[r] = o_lse;
    q.tlogit[r] = o_tl;
    q.ce[r] = o_ce;
    q.ent[r] = o_ent;
    q.amax[r] = o_am;
    q.cew_out[r] = o_cw;
    if (q.top != nullptr) q.top[r] = o_top;
  }
  if (drow != nullptr && dx_mode != DX_FINISH) {
    const float* src = dx_mode == DX_COPY ? q.dxc + static_cast<size_t>(pos) * q.h : nullptr;
    for (int c = threadIdx.x * 4; c < q.h; c += 128 * 4)
      *reinterpret_cast<float4*>(drow + c) =
          src != nullptr ? *reinterpret_cast<const float4*>(src + c) : make_float4(0.f, 0.f, 0.f, 0.f);
  }
}

// One block, fixed reduction order: the loss and the step's scalars (MET_*). A non-zero device
// status poisons the loss so a failed sweep cannot pass for a result.
// Replaces op.py:127 and the counters of patch.py:480-486 / the sums behind patch.py:582-615.
__global__ void __launch_bounds__(1024)
head_step_scalars_kernel(int m, long long v, const float* __restrict__ ce,
                         const float* __restrict__ cew, const float* __restrict__ ent,
                         const long long* __restrict__ amax, const long long* __restrict__ tgt_o,
                         const long long* __restrict__ attn, const int* __restrict__ counts,
                         const int* __restrict__ status, float* __restrict__ loss,
                         float* __restrict__ metrics) {
  __shared__ double sh[7][32];
  double a[7] = {0.0, 0.0, 0.0, 0.0, 0.0, 0.0, 0.0};
  for (int i = threadIdx.x; i < m; i += blockDim.x) {
    const long long tg = tgt_o[i];
    const bool valid = tg >= 0 && tg < v;
    a[MET_LOSS] += static_cast<double>(cew[i]) * static_cast<double>(ce[i]);
    if (valid) {
      a[MET_VALID] += 1.0;
      a[MET_CORRECT] += (amax[i] == tg) ? 1.0 : 0.0;
      a[MET_ENT_VALID] += static_cast<double>(ent[i]);
    }
    if (tg != -100) a[MET_LABELLED] += 1.0;
    if (attn == nullptr || attn[i] != 0) {
      a[MET_ATTENDED] += 1.0;
      a[MET_ENT_ATT] += static_cast<double>(ent[i]);
    }
  }
#pragma unroll
  for (int k = 0; k < 7; ++k)
    for (int o = 16; o > 0; o >>= 1) a[k] += __shfl_xor_sync(0xffffffffu, a[k], o);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  if (l == 0)
    for (int k = 0; k < 7; ++k) sh[k][w] = a[k];
  __syncthreads();
  if (threadIdx.x == 0) {
    const int nw = blockDim.x >> 5;
    double r[7] = {0.0, 0.0, 0.0, 0.0, 0.0, 0.0, 0.0};
    for (int i = 0; i < nw; ++i)
      for (int k = 0; k < 7; ++k) r[k] += sh[k][i];
    float lo = static_cast<float>(r[MET_LOSS]);
    if (status != nullptr && *status != 0) lo = __int_as_float(0x7fc00000);
    loss[0] = lo;
    if (metrics != nullptr) {
      metrics[MET_LOSS] = lo;
      for (int k = 1; k < 7; ++k) metrics[k] = static_cast<float>(r[k]);
      metrics[MET_LIVE] = static_cast<float>(counts[CNT_LIVE]);
    }
  }
}

}  // namespace esep
