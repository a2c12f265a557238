// The head weight's storage format: ONE fp16 tensor shared by the LM head and the embedding
// lookup, plus the table of elements that fp16 does not hold exactly.
//
// Replaces the reference's torch code for that format (solution/head/patch.py:133-215,
// _Fp16Fixup, and :217-226, _embedding_forward16): the head reads the fp16 tensor as it is; the
// embedding lookup must return the fp32 values of the original weight bit for bit, so it gathers
// fp16 rows, upcasts them and writes back the exact fp32 value of every element that does not
// survive fp32 -> fp16 -> fp32 (values under fp16's normal range, overflows, NaN payloads).
//
// The table is kept in compressed rows (row_start[v + 1], and per entry the flat element index and
// the exact fp32 value, sorted by index) instead of the reference's padded per-row matrices: a
// lookup needs no fixed shape here because it happens inside the gather kernel. All kernels are
// HBM bound:
//   scan     4 B read + 2 B written per weight element (one pass: cast and count together)
//   fill     touches only the rows that have entries
//   embed    2 H read + 4 H written per looked-up row, + its entries
//   exact    2 B read + 4 B written per element, + the entries
#pragma once

#include <cuda_fp16.h>

#include "head_norm.cuh"

namespace esep {

__device__ __forceinline__ bool fp16_round_trip_differs(float x, __half hx) {
  return __float_as_uint(__half2float(hx)) != __float_as_uint(x);
}

// One block of 128 threads per weight row, every thread's loads issued before any is used (the
// shape of the norm kernels, which run at the copy bandwidth). kCast: w16 is written (round to
// nearest even, the conversion torch uses on the device); otherwise w16 is the caller's tensor
// and only compared. counts[row] = elements of the row whose fp16 value does not give back the
// fp32 bits; stats (zeroed before the launch): stats[3 + b] = entries of rows [1024 b, 1024 b + 1024).
template <bool kCast>
__global__ void __launch_bounds__(128)
head_w16_scan_kernel(const float* __restrict__ w32, __half* w16, int v, int h,
                     int* __restrict__ counts, long long* stats) {
  __shared__ int sh[4];
  const int row = blockIdx.x;
  const size_t base = static_cast<size_t>(row) * h;
  int bad = 0;
  for (int c0 = threadIdx.x * 4; c0 < h; c0 += 2048) {   // h % 4 == 0
    float4 x[4];
    uint2 raw[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int c = c0 + u * 512;
      if (c < h) {
        x[u] = *reinterpret_cast<const float4*>(w32 + base + c);
        if (!kCast) raw[u] = *reinterpret_cast<const uint2*>(w16 + base + c);
      }
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int c = c0 + u * 512;
      if (c < h) {
        __half2 lo, hi;
        if (kCast) {
          lo = __floats2half2_rn(x[u].x, x[u].y);
          hi = __floats2half2_rn(x[u].z, x[u].w);
          uint2 out;
          out.x = *reinterpret_cast<const uint32_t*>(&lo);
          out.y = *reinterpret_cast<const uint32_t*>(&hi);
          *reinterpret_cast<uint2*>(w16 + base + c) = out;
        } else {
          lo = *reinterpret_cast<const __half2*>(&raw[u].x);
          hi = *reinterpret_cast<const __half2*>(&raw[u].y);
        }
        bad += fp16_round_trip_differs(x[u].x, __low2half(lo)) +
               fp16_round_trip_differs(x[u].y, __high2half(lo)) +
               fp16_round_trip_differs(x[u].z, __low2half(hi)) +
               fp16_round_trip_differs(x[u].w, __high2half(hi));
      }
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) bad += __shfl_xor_sync(0xffffffffu, bad, o);
  if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = bad;
  __syncthreads();
  if (threadIdx.x == 0) {
    bad = sh[0] + sh[1] + sh[2] + sh[3];
    counts[row] = bad;
    if (bad > 0)   // entries per block of 1024 rows (integers: the order does not matter)
      atomicAdd(reinterpret_cast<unsigned long long*>(stats + 3 + (row >> 10)),
                static_cast<unsigned long long>(bad));
  }
}

// In place: counts[0 .. v) -> exclusive prefix, row_start[v] = total. Block b owns rows
// [1024 b, 1024 b + 1024): its base is the sum of the earlier blocks' entries (stats[3 ..]).
// Also leaves stats[0 .. 3) = {entries, rows with entries, most entries in one row}.
__global__ void __launch_bounds__(1024)
head_w16_offsets_kernel(int* row_start, int v, long long* stats) {
  __shared__ int sh[32];
  __shared__ int sh_base;
  const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
  int part = 0;
  for (int b = t; b < static_cast<int>(blockIdx.x); b += 1024) part += static_cast<int>(stats[3 + b]);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) part += __shfl_xor_sync(0xffffffffu, part, o);
  if (lane == 0) sh[warp] = part;
  __syncthreads();
  if (t == 0) {
    int base = 0;
    for (int w = 0; w < 32; ++w) base += sh[w];
    sh_base = base;
  }
  __syncthreads();
  const int row = blockIdx.x * 1024 + t;
  const int c = row < v ? row_start[row] : 0;
  int incl = c;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int u = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += u;
  }
  __syncthreads();   // sh is reused
  if (lane == 31) sh[warp] = incl;
  __syncthreads();
  if (warp == 0) {
    int ws = sh[lane];
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int u = __shfl_up_sync(0xffffffffu, ws, o);
      if (lane >= o) ws += u;
    }
    sh[lane] = ws;   // inclusive over warps
  }
  __syncthreads();
  const int excl = sh_base + (warp > 0 ? sh[warp - 1] : 0) + incl - c;
  if (row < v) row_start[row] = excl;
  if (row == v - 1) {
    row_start[v] = excl + c;
    stats[0] = excl + c;
  }
  // rows with entries and the most entries in one row: one pair of atomics per block
  int rows = c > 0, mx = c;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    rows += __shfl_xor_sync(0xffffffffu, rows, o);
    mx = max(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  }
  if (lane == 0 && rows > 0) {
    atomicAdd(reinterpret_cast<unsigned long long*>(stats + 1), static_cast<unsigned long long>(rows));
    atomicMax(stats + 2, static_cast<long long>(mx));
  }
}

// One block of 128 threads per row; rows without entries leave at once. The entries come out in
// column order, so the table is sorted by flat index (the order of the reference's nonzero(),
// patch.py:145): a thread takes four adjacent columns of every 512-column step, and within a step
// that has entries their places follow from a prefix sum over the block.
__global__ void __launch_bounds__(128)
head_w16_fill_kernel(const float* __restrict__ w32, const __half* __restrict__ w16, int v, int h,
                     const int* __restrict__ row_start, long long* __restrict__ flat_idx,
                     float* __restrict__ flat_val) {
  __shared__ int sh[4];
  const int row = blockIdx.x;
  int pos = row_start[row];
  if (row_start[row + 1] == pos) return;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const size_t base = static_cast<size_t>(row) * h;
  for (int c0 = 0; c0 < h; c0 += 512) {
    const int c = c0 + threadIdx.x * 4;
    float x[4] = {0.f, 0.f, 0.f, 0.f};
    bool bad[4] = {false, false, false, false};
    if (c < h) {   // h % 4 == 0
      const float4 xv = *reinterpret_cast<const float4*>(w32 + base + c);
      const uint2 raw = *reinterpret_cast<const uint2*>(w16 + base + c);
      const __half2 lo = *reinterpret_cast<const __half2*>(&raw.x);
      const __half2 hi = *reinterpret_cast<const __half2*>(&raw.y);
      x[0] = xv.x; x[1] = xv.y; x[2] = xv.z; x[3] = xv.w;
      bad[0] = fp16_round_trip_differs(xv.x, __low2half(lo));
      bad[1] = fp16_round_trip_differs(xv.y, __high2half(lo));
      bad[2] = fp16_round_trip_differs(xv.z, __low2half(hi));
      bad[3] = fp16_round_trip_differs(xv.w, __high2half(hi));
    }
    const int mine = bad[0] + bad[1] + bad[2] + bad[3];
    if (!__syncthreads_or(mine != 0)) continue;
    int incl = mine;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int u = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += u;
    }
    if (lane == 31) sh[warp] = incl;
    __syncthreads();
    int before = 0, total = 0;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      if (w < warp) before += sh[w];
      total += sh[w];
    }
    int at = pos + before + incl - mine;
#pragma unroll
    for (int j = 0; j < 4; ++j)
      if (bad[j]) {
        flat_idx[at] = static_cast<long long>(base + c + j);
        flat_val[at] = x[j];
        ++at;
      }
    pos += total;
    __syncthreads();   // sh is reused by the next step
  }
}

// out[i, :] = exact fp32 row ids[i] of the original weight. One block of 128 threads per looked-up
// row. w16 == nullptr: out already holds the upcast rows and only the entries are written (the
// reference's apply_rows, patch.py:201-210). An id outside [0, v) gives a zero row and sets *status.
__global__ void __launch_bounds__(128)
head_embed_rows_kernel(const __half* __restrict__ w16, const long long* __restrict__ ids, int v,
                       int h, const int* __restrict__ row_start,
                       const long long* __restrict__ flat_idx, const float* __restrict__ flat_val,
                       float* __restrict__ out, int* status) {
  const long long id = ids[blockIdx.x];
  float* dst = out + static_cast<size_t>(blockIdx.x) * h;
  if (id < 0 || id >= v) {
    if (w16 != nullptr)
      for (int c = threadIdx.x * 4; c < h; c += 512)
        *reinterpret_cast<float4*>(dst + c) = make_float4(0.f, 0.f, 0.f, 0.f);
    if (threadIdx.x == 0 && status != nullptr) atomicCAS(status, DEV_OK, DEV_BAD_INDEX);
    return;
  }
  const size_t base = static_cast<size_t>(id) * h;
  if (w16 != nullptr) {
    for (int c = threadIdx.x * 8; c < h; c += 1024) {   // h % 8 == 0
      const uint4 raw = *reinterpret_cast<const uint4*>(w16 + base + c);
      const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&raw.x));
      const float2 b = __half22float2(*reinterpret_cast<const __half2*>(&raw.y));
      const float2 e = __half22float2(*reinterpret_cast<const __half2*>(&raw.z));
      const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&raw.w));
      *reinterpret_cast<float4*>(dst + c) = make_float4(a.x, a.y, b.x, b.y);
      *reinterpret_cast<float4*>(dst + c + 4) = make_float4(e.x, e.y, f.x, f.y);
    }
  }
  if (row_start == nullptr) return;
  const int e0 = row_start[id], e1 = row_start[id + 1];
  if (e0 == e1) return;
  __syncthreads();   // the entries overwrite what the loop above stored
  for (int e = e0 + threadIdx.x; e < e1; e += 128)
    dst[flat_idx[e] - static_cast<long long>(base)] = flat_val[e];
}

// out = fp32 copy of w16 (the entries are written by head_w16_restore_kernel afterwards). A block
// converts 1024 consecutive 16-byte groups; every thread's four loads are issued first.
__global__ void __launch_bounds__(256)
head_w16_upcast_kernel(const __half* __restrict__ w16, size_t n8, float* __restrict__ out) {
  const size_t i0 = static_cast<size_t>(blockIdx.x) * 1024 + threadIdx.x;
  uint4 raw[4];
#pragma unroll
  for (int u = 0; u < 4; ++u)
    if (i0 + u * 256 < n8) raw[u] = reinterpret_cast<const uint4*>(w16)[i0 + u * 256];
#pragma unroll
  for (int u = 0; u < 4; ++u) {
    const size_t i = i0 + u * 256;
    if (i < n8) {
      const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&raw[u].x));
      const float2 b = __half22float2(*reinterpret_cast<const __half2*>(&raw[u].y));
      const float2 e = __half22float2(*reinterpret_cast<const __half2*>(&raw[u].z));
      const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&raw[u].w));
      reinterpret_cast<float4*>(out)[2 * i] = make_float4(a.x, a.y, b.x, b.y);
      reinterpret_cast<float4*>(out)[2 * i + 1] = make_float4(e.x, e.y, f.x, f.y);
    }
  }
}

__global__ void __launch_bounds__(256)
head_w16_restore_kernel(const long long* __restrict__ flat_idx, const float* __restrict__ flat_val,
                        long long count, float* __restrict__ out) {
  const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i < count) out[flat_idx[i]] = flat_val[i];
}

}  // namespace esep
