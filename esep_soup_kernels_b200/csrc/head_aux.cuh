// Small memory-bound kernels around the two tensor-core sweeps: merging partial softmax records,
// per-row outputs, the scalar loss / metric reduction and the sum of partial dHidden buffers.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "head_fwd.cuh"

namespace esep {

// Merges K partial records per row with the rule of solution/head/kernels.py:70-75:
//   M = max m_k ; S = sum s_k e^(m_k - M) ; T = sum e^(m_k - M) (t_k + s_k (m_k - M))
//   tz = sum tz_k (only the owner of the target contributed) ; idx = idx_k of the FIRST k with
//   m_k == M  (partials are ordered by ascending vocabulary range, so this is the lowest index)
// Input arrays are [K][n]; `idx_offset` is added to the index (local -> global id).
__global__ void head_merge_kernel(int n, int k_parts, const float* __restrict__ pm,
                                  const float* __restrict__ ps, const float* __restrict__ pt,
                                  const float* __restrict__ ptz, const int* __restrict__ pidx,
                                  long long idx_offset, float* __restrict__ record,
                                  const int* gate = nullptr) {
  const int row = blockIdx.x * blockDim.x + threadIdx.x;
  if (row >= n || (gate != nullptr && *gate == 0)) return;
  float big = NEG_BIG;
  for (int k = 0; k < k_parts; ++k) big = fmaxf(big, pm[static_cast<size_t>(k) * n + row]);
  float s = 0.f, t = 0.f, tz = 0.f;
  int idx = 0;
  bool found = false;
  for (int k = 0; k < k_parts; ++k) {
    const size_t o = static_cast<size_t>(k) * n + row;
    const float mk = pm[o];
    const float dl = mk - big;
    const float sc = __expf(dl);
    const float sk = ps[o];
    s += sk * sc;
    t += sc * (pt[o] + sk * dl);
    tz += ptz[o];
    if (!found && mk == big) {
      found = true;
      idx = pidx[o];
    }
  }
  record[0 * static_cast<size_t>(n) + row] = big;
  record[1 * static_cast<size_t>(n) + row] = s;
  record[2 * static_cast<size_t>(n) + row] = t;
  record[3 * static_cast<size_t>(n) + row] = tz;
  record[4 * static_cast<size_t>(n) + row] =
      __int_as_float(static_cast<int>(idx + idx_offset));
}

// records: [K][5][n] (K = 1 on one GPU). Writes the per-row outputs of the op
// (solution/head/op.py:125-126: target_logit and ce are 0 on ignored rows; lse / entropy /
// argmax exist for every row) and the masked weight (op.py:105-107).
__global__ void head_rows_kernel(int n, int k_parts, long long v_global,
                                 const float* __restrict__ records,
                                 const long long* __restrict__ target,
                                 const float* __restrict__ ce_weight, float* __restrict__ lse,
                                 float* __restrict__ tlogit, float* __restrict__ ce,
                                 float* __restrict__ ent, long long* __restrict__ amax,
                                 float* __restrict__ cew_out, const int* gate = nullptr) {
  const int row = blockIdx.x * blockDim.x + threadIdx.x;
  if (row >= n || (gate != nullptr && *gate == 0)) return;
  const size_t stride = 5 * static_cast<size_t>(n);
  float big = NEG_BIG;
  for (int k = 0; k < k_parts; ++k) big = fmaxf(big, records[k * stride + row]);
  float s = 0.f, t = 0.f, tz = 0.f;
  int idx = 0x7fffffff;
  for (int k = 0; k < k_parts; ++k) {
    const float* r = records + k * stride;
    const float mk = r[row];
    const float dl = mk - big;
    const float sc = __expf(dl);
    const float sk = r[n + row];
    s += sk * sc;
    t += sc * (r[2 * static_cast<size_t>(n) + row] + sk * dl);
    tz += r[3 * static_cast<size_t>(n) + row];
    if (mk == big) idx = min(idx, __float_as_int(r[4 * static_cast<size_t>(n) + row]));
  }
  const float log_s = logf(s);
  const float l = big + log_s;
  const long long tg = target[row];
  const bool valid = tg >= 0 && tg < v_global;
  lse[row] = l;
  ent[row] = log_s - t / s;
  amax[row] = idx;
  tlogit[row] = valid ? tz : 0.f;
  ce[row] = valid ? (l - tz) : 0.f;
  cew_out[row] = valid ? ce_weight[row] : 0.f;
}

// One block, fixed reduction order: loss = sum cew * ce and the metric scalars
// {loss, n_valid, n_correct, sum of entropy over valid rows}. A non-zero device status
// poisons the loss so a failed sweep cannot pass for a result.
__global__ void head_scalars_kernel(int n, long long v_global, const float* __restrict__ ce,
                                    const float* __restrict__ cew, const float* __restrict__ ent,
                                    const long long* __restrict__ amax,
                                    const long long* __restrict__ target,
                                    const int* __restrict__ status, float* __restrict__ loss,
                                    float* __restrict__ metrics, const int* gate = nullptr) {
  __shared__ double sh[4][32];
  if (gate != nullptr && *gate == 0) return;
  double a0 = 0.0, a1 = 0.0, a2 = 0.0, a3 = 0.0;
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const long long tg = target[i];
    const bool valid = tg >= 0 && tg < v_global;
    a0 += static_cast<double>(cew[i]) * static_cast<double>(ce[i]);
    if (valid) {
      a1 += 1.0;
      a2 += (amax[i] == tg) ? 1.0 : 0.0;
      a3 += static_cast<double>(ent[i]);
    }
  }
  for (int o = 16; o > 0; o >>= 1) {
    a0 += __shfl_xor_sync(0xffffffffu, a0, o);
    a1 += __shfl_xor_sync(0xffffffffu, a1, o);
    a2 += __shfl_xor_sync(0xffffffffu, a2, o);
    a3 += __shfl_xor_sync(0xffffffffu, a3, o);
  }
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  if (l == 0) {
    sh[0][w] = a0;
    sh[1][w] = a1;
    sh[2][w] = a2;
    sh[3][w] = a3;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    double r0 = 0.0, r1 = 0.0, r2 = 0.0, r3 = 0.0;
    const int nw = blockDim.x >> 5;
    for (int i = 0; i < nw; ++i) {
      r0 += sh[0][i];
      r1 += sh[1][i];
      r2 += sh[2][i];
      r3 += sh[3][i];
    }
    float lo = static_cast<float>(r0);
    if (status != nullptr && *status != 0) lo = __int_as_float(0x7fc00000);
    loss[0] = lo;
    if (metrics != nullptr) {
      metrics[0] = lo;
      metrics[1] = static_cast<float>(r1);
      metrics[2] = static_cast<float>(r2);
      metrics[3] = static_cast<float>(r3);
    }
  }
}

// Adds up the partial dHidden pieces of the left-over (row tile, pass) pairs, in vocabulary
// order, and writes them into dx. Piece q of pair j sits in part[q][j][128][pass_width].
// One block per (pair, row of the tile).
__global__ void head_dx_sum_kernel(int n, int h, int n_row_tiles, int first_tp, int rem_tp,
                                   int pieces, int pass_width, const float* __restrict__ part,
                                   float* __restrict__ dx, const int* gate = nullptr) {
  if (gate != nullptr && *gate == 0) return;
  const int j = blockIdx.x / 128, rr = blockIdx.x % 128;
  const int tp = first_tp + j;
  const int row = (tp % n_row_tiles) * 128 + rr;
  if (row >= n) return;
  const int col0 = (tp / n_row_tiles) * pass_width;
  const size_t piece_stride = static_cast<size_t>(rem_tp) * 128 * pass_width;
  const float* src = part + (static_cast<size_t>(j) * 128 + rr) * pass_width;
  for (int cidx = threadIdx.x * 4; cidx < pass_width && col0 + cidx < h; cidx += blockDim.x * 4) {
    float4 a = *reinterpret_cast<const float4*>(src + cidx);
    for (int q = 1; q < pieces; ++q) {
      const float4 b = *reinterpret_cast<const float4*>(src + q * piece_stride + cidx);
      a.x += b.x;
      a.y += b.y;
      a.z += b.z;
      a.w += b.w;
    }
    *reinterpret_cast<float4*>(dx + static_cast<size_t>(row) * h + col0 + cidx) = a;
  }
}

// ---- vocabulary shards that each ran the single pass as a vocabulary of their own ----------------
// Every shard k sweeps its rows of W with a LOCAL softmax: local lse_k, local entropy H_k, its
// largest logit and where it sits, the target logit on the shard that owns the target, and
// dX_k = p_k W_k - W_k[t_k] for a local target t_k with unit weight. The global results follow
// from one exchange of five numbers per row and shard:
//     lse = logsumexp_k lse_k        a_k = e^(lse_k - lse)      (softmax = a_k p_k on shard k)
//     entropy = lse - sum_k a_k (lse_k - H_k)
//     argmax: the shard whose largest logit is largest, lowest global index on equal values
//     dX = cew (sum_k a_k p_k W_k - W[target])
// Rows whose target lives on another shard sweep with local target 0 as a stand-in and the row
// W_k[0] is added back; on the owner the two target terms combine to -(1 - a_k) W[target], with
// 1 - a_k formed from the OTHER shards' a so that a confident row loses nothing to cancellation.

// Local target and unit weight of every row for the shard [vocab_offset, vocab_offset + v_local).
__global__ void head_vp_prepare_kernel(int n, long long v_global, long long vocab_offset,
                                       long long v_local, const long long* __restrict__ target,
                                       long long* __restrict__ local_target,
                                       float* __restrict__ unit_weight) {
  const int row = blockIdx.x * blockDim.x + threadIdx.x;
  if (row >= n) return;
  const long long tg = target[row];
  const bool valid = tg >= 0 && tg < v_global;
  const long long tl = tg - vocab_offset;
  const bool owner = valid && tl >= 0 && tl < v_local;
  local_target[row] = owner ? tl : (valid ? 0 : -100);
  unit_weight[row] = valid ? 1.f : 0.f;
}

// The record a shard sends: [5][n] = lse_k, H_k, largest logit, target logit (owner only, else
// 0), global index of the largest logit (an int32 stored bit for bit).
__global__ void head_vp_pack_kernel(int n, long long v_global, long long vocab_offset,
                                    long long v_local, const long long* __restrict__ target,
                                    const float* __restrict__ lse, const float* __restrict__ ent,
                                    const float* __restrict__ top,
                                    const float* __restrict__ tlogit,
                                    const long long* __restrict__ amax_local,
                                    float* __restrict__ record) {
  const int row = blockIdx.x * blockDim.x + threadIdx.x;
  if (row >= n) return;
  const long long tg = target[row];
  const long long tl = tg - vocab_offset;
  const bool owner = tg >= 0 && tg < v_global && tl >= 0 && tl < v_local;
  const size_t ns = static_cast<size_t>(n);
  record[row] = lse[row];
  record[ns + row] = ent[row];
  record[2 * ns + row] = top[row];
  record[3 * ns + row] = owner ? tlogit[row] : 0.f;
  record[4 * ns + row] = __int_as_float(static_cast<int>(amax_local[row] + vocab_offset));
}

struct VpCombineParams {
  int n, h, k_parts, me;
  long long v_global, vocab_offset, v_local;
  const float* records;        // [k_parts][5][n], shard order
  const long long* target;     // [n] global ids
  const float* ce_weight;      // [n]
  const void* w_shard;         // [v_local, h]
  float* dx;                   // [n, h] in: the local sweep's dX_k (unit weight); out: this shard's
                               // share of dHidden
  float *lse, *tlogit, *ce, *ent, *cew_out;
  long long* amax;
};

// One block of 128 threads per row; every thread forms the row's scalars itself (k_parts is
// small), then the block rewrites the row of dx in place.
template <int kFmt>
__global__ void __launch_bounds__(128) head_vp_combine_kernel(const VpCombineParams q) {
  const int row = blockIdx.x;
  const size_t ns = static_cast<size_t>(q.n);
  const size_t stride = 5 * ns;
  float big = NEG_BIG;
  for (int k = 0; k < q.k_parts; ++k) big = fmaxf(big, q.records[k * stride + row]);
  float se = 0.f;
  for (int k = 0; k < q.k_parts; ++k) se += __expf(q.records[k * stride + row] - big);
  const float lse = big + logf(se);
  float mix = 0.f, tz = 0.f, best = -INFINITY, a_me = 0.f, a_rest = 0.f;
  int idx = 0x7fffffff;
  for (int k = 0; k < q.k_parts; ++k) {
    const float* r = q.records + k * stride;
    const float lk = r[row];
    const float ak = __expf(lk - lse);
    mix += ak * (lk - r[ns + row]);
    tz += r[3 * ns + row];
    const float tk = r[2 * ns + row];
    const int ik = __float_as_int(r[4 * ns + row]);
    if (tk > best || (tk == best && ik < idx)) {
      best = tk;
      idx = ik;
    }
    if (k == q.me) a_me = ak; else a_rest += ak;
  }
  const long long tg = q.target[row];
  const bool valid = tg >= 0 && tg < q.v_global;
  const float cw = valid ? q.ce_weight[row] : 0.f;
  if (threadIdx.x == 0) {
    q.lse[row] = lse;
    q.ent[row] = lse - mix;
    q.amax[row] = idx;
    q.tlogit[row] = valid ? tz : 0.f;
    q.ce[row] = valid ? (lse - tz) : 0.f;
    q.cew_out[row] = cw;
  }
  const long long tl = tg - q.vocab_offset;
  const bool owner = valid && tl >= 0 && tl < q.v_local;
  // a p_k W_k - a W_k[t_k] + coef W_k[t_k]: coef = a on a stand-in target (adds the row back),
  // -(1 - a) on the owner (the rest of the -W[target] term)
  const float coef = owner ? -a_rest : a_me;
  const size_t wrow = static_cast<size_t>(owner ? tl : 0) * q.h;
  float* drow = q.dx + static_cast<size_t>(row) * q.h;
  for (int c = threadIdx.x * 4; c < q.h; c += 128 * 4) {
    float4 val = make_float4(0.f, 0.f, 0.f, 0.f);
    if (cw != 0.f) {
      const float4 d = *reinterpret_cast<const float4*>(drow + c);
      const uint2 raw = reinterpret_cast<const uint2*>(q.w_shard)[(wrow + c) / 4];
      float2 w01, w23;
      if (kFmt == 0) {
        w01 = __half22float2(*reinterpret_cast<const __half2*>(&raw.x));
        w23 = __half22float2(*reinterpret_cast<const __half2*>(&raw.y));
      } else {
        w01 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
        w23 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
      }
      val = make_float4(cw * (a_me * d.x + coef * w01.x), cw * (a_me * d.y + coef * w01.y),
                        cw * (a_me * d.z + coef * w23.x), cw * (a_me * d.w + coef * w23.y));
    }
    *reinterpret_cast<float4*>(drow + c) = val;
  }
}

// out[i] = dx[i] * grad_loss[0], stored as fp16 (0), bf16 (1) or fp32 (2): the whole autograd
// backward of the op (solution/head/op.py:143-145) in one pass, grad_loss read on the device.
template <int kOut>
__global__ void __launch_bounds__(256)
head_grad_scale_kernel(const float4* __restrict__ dx, const float* __restrict__ grad_loss,
                       long long n4, void* __restrict__ out) {
  const float g = grad_loss[0];
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n4;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    float4 v = dx[i];
    v.x *= g;
    v.y *= g;
    v.z *= g;
    v.w *= g;
    if (kOut == 2) {
      reinterpret_cast<float4*>(out)[i] = v;
    } else if (kOut == 0) {
      const __half2 a = __floats2half2_rn(v.x, v.y), b = __floats2half2_rn(v.z, v.w);
      reinterpret_cast<uint2*>(out)[i] = make_uint2(*reinterpret_cast<const uint32_t*>(&a),
                                                   *reinterpret_cast<const uint32_t*>(&b));
    } else {
      const __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
      reinterpret_cast<uint2*>(out)[i] = make_uint2(*reinterpret_cast<const uint32_t*>(&a),
                                                   *reinterpret_cast<const uint32_t*>(&b));
    }
  }
}

// Exercises the bounded-wait path on purpose: one warp waits on an mbarrier that nothing ever
// arrives on, gives up after `limit_cycles`, records DEV_TIMEOUT_SELFTEST in the status word and
// returns normally (no trap, the context stays usable). Used by the test suite only.
enum : int { DEV_TIMEOUT_SELFTEST = 901 };
__global__ void head_wait_probe_kernel(int* status, long long limit_cycles) {
  __shared__ __align__(8) unsigned long long bar_storage;
  __shared__ int abort_flag;
  const uint32_t bar = smem_u32(&bar_storage);
  if (threadIdx.x == 0) {
    mbar_init(bar, 1);
    abort_flag = 0;
    fence_barrier_init();
  }
  __syncthreads();
  const bool ok = __all_sync(0xffffffffu, mbar_wait(bar, 0, &abort_flag, limit_cycles));
  if (!ok && threadIdx.x == 0) atomicCAS(status, DEV_OK, DEV_TIMEOUT_SELFTEST);
}

}  // namespace esep
