// Forward sweep of the LM head: logits tiles on tcgen05 tensor cores, softmax statistics in the
// epilogue; the statistics-only form never lets a logit leave the SM.
//
// Replaces, for all rows of x, the per-chunk pair
//     torch.mm(x16[r0:r0+nr], W.t(), out=z)                    (solution/head/op.py:90)
//     head_row_softmax_kernel pass 1                           (solution/head/kernels.py:46-82)
// of the reference. Two CTAs work as a pair (cta_group::2, MMA M = 256): one work unit = (two
// 128-row tiles of x, one per CTA) x (a run of 256-wide vocabulary tiles). Each CTA loads its own
// x tile and HALF of every W tile (128 of the 256 vocabulary rows), which cuts the L2 -> shared
// memory traffic per tile from 1.18 MB to 0.79 MB per SM. For each vocabulary tile every CTA gets
// the 128x256 fp32 logits of its rows in tensor memory (TMEM); four epilogue warps read them back
// one 32-column chunk at a time (thread = row) and fold them into the running per-row record
//     m  = max z          s = sum e^(z-m)        t = sum e^(z-m) (z-m)
//     i  = first index of the max                tz = z[target]
// with the update rule of kernels.py:59-68. The record of each unit is written to a small
// per-(split,row) scratch array; head_finalize merges the splits with the rule of
// kernels.py:70-81 (lse = M + ln S, entropy = ln S - T/S, argmax = lowest index of the max).
//
// Warp roles (192 threads): warp 0 = TMA producer (both CTAs), warp 1 = MMA issuer (pair leader
// only) + TMEM owner, warps 2..5 = epilogue (TMEM lane quadrant = warp_id % 4). The TMEM
// accumulator is double buffered (2 x 256 columns) so the MMAs of tile k+1 overlap the epilogue
// of tile k.
//
// kStore launches are the first of the training path's two sweeps (head_dx.cuh is the second):
// they also keep one 16-bit value per logit in HBM - kStore 1: fp16 (z - m_ref) log2 e written
// straight from the registers; kStore 2: the bf16 softmax weight 2^((z - m_ref - 40) log2 e), zero
// at the target, which each epilogue warp stages in shared memory as a swizzled 64 x 32 box and
// stores with one TMA instruction - and leave the target's entry out of the row sums.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "sm100_ptx.cuh"

namespace esep {

static constexpr float NEG_BIG = -1.0e30f;  // finite "minus infinity" (kernels.py:33-34)
static constexpr float LOG2E = 1.4426950408889634f;
static constexpr float LN2 = 0.6931471805599453f;

// Error codes a kernel can leave in the device status word.
enum : int {
  DEV_OK = 0,
  DEV_TIMEOUT_PRODUCER = 101,
  DEV_TIMEOUT_MMA = 102,
  DEV_TIMEOUT_EPILOGUE = 103,
  DEV_BAD_INDEX = 301,   // an embedding id outside the vocabulary (head_embed_rows_kernel)
};

struct FwdParams {
  int n;               // rows of x
  int h;               // hidden size (K)
  int v;               // vocabulary rows in this W (local V)
  int n_row_tiles;     // ceil(n / 128)
  int n_row_pairs;     // ceil(n_row_tiles / 2): a CTA pair sweeps two row tiles at once
  int n_vtiles;        // ceil(v / 256)
  int tiles_per_unit;  // vocabulary tiles per work unit
  int n_splits;        // ceil(n_vtiles / tiles_per_unit)
  long long vocab_offset;  // global id of local vocabulary row 0 (vocab-parallel shards)
  const long long* target;  // [n] global ids; anything outside this shard never matches
  float* pm;           // [n_splits, n] partial max
  float* ps;           // [n_splits, n] partial sum exp
  float* pt;           // [n_splits, n] partial sum exp * (z - m)
  float* ptz;          // [n_splits, n] partial target logit (0 unless the shard/split owns it)
  int* pidx;           // [n_splits, n] local index of the partial max
  int* status;         // device status word
  const int* gate;     // null, or a device flag: the kernel does nothing when it reads 0
  // Rows known only on the device: when `row_range` is set the kernel sweeps the rows
  // [row_range[0], row_range[1]) of x (both read on the device, end <= n) and derives its own
  // work split from their number (fwd_split_rows); partial records then sit at
  // [split][row - row_range[0]] with a stride of fwd_split_rows().stride.
  const int* row_range;
  int part_cap;        // rows the partial arrays hold (splits * stride never exceeds it)
  // kStore launches only (the sweep that keeps the logits for the dHidden kernel, head_dx.cuh):
  // zbuf[row - row_range[0]][vocab] = fp16((logit - m_ref[row]) * log2 e) with `zpitch` elements per row
  // (a multiple of 256, so that whole tiles can be stored); the row sums then leave the
  // target's own entry out, as the training sweeps do (it is added in fp32 by the row finish).
  // kStore == 2 keeps the softmax weights themselves instead: bf16(2^((logit - m_ref - 40) log2 e)),
  // zero at the target's entry and past the end of the vocabulary, so that the dHidden kernel can
  // take its tiles straight from this buffer (bf16 has fp32's exponent range: see m_ref's margin).
  __half* zbuf;
  long long zpitch;
  const float* m_ref;
};

// Work split of the forward sweep for a row count that is only known on the device: the
// vocabulary tiles of every row pair are cut into `splits` runs of `tiles_per_unit` tiles so
// that the units fill the resident CTA pairs evenly (the first split count that reaches 97 %,
// else the best), subject to splits * stride <= part_cap. Cheap enough for every thread.
struct FwdSplit {
  int n_row_tiles, n_row_pairs, tiles_per_unit, n_splits, stride;
};
__host__ __device__ inline FwdSplit fwd_split_rows(int n_rows, int n_vtiles, int n_pairs,
                                                   int part_cap) {
  FwdSplit r;
  r.n_row_tiles = (n_rows + 127) / 128;
  r.n_row_pairs = (r.n_row_tiles + 1) / 2;
  r.stride = r.n_row_pairs * 256;
  r.tiles_per_unit = n_vtiles > 0 ? n_vtiles : 1;
  r.n_splits = 1;
  if (r.n_row_pairs <= 0 || n_vtiles <= 0) {
    r.n_splits = 0;
    return r;
  }
  if (n_pairs < 1) n_pairs = 1;
  int max_splits = r.stride > 0 ? part_cap / r.stride : 1;
  if (max_splits > 128) max_splits = 128;
  if (max_splits > n_vtiles) max_splits = n_vtiles;
  const float ideal = static_cast<float>(r.n_row_pairs) * n_vtiles / n_pairs;
  float best = -1.f;
  for (int want = 1; want <= max_splits; ++want) {
    const int tpu = (n_vtiles + want - 1) / want;
    const int splits = (n_vtiles + tpu - 1) / tpu;
    const int waves = (r.n_row_pairs * splits + n_pairs - 1) / n_pairs;
    const float eff = ideal / (static_cast<float>(waves) * tpu);
    if (eff > best + 1e-6f) {
      best = eff;
      r.tiles_per_unit = tpu;
      r.n_splits = splits;
    }
    if (eff >= 0.97f) break;
  }
  return r;
}

namespace fwd {
static constexpr int BM = 128;      // rows per tile (TMEM lanes)
static constexpr int BN = 256;      // vocabulary columns per tile (MMA N)
static constexpr int BK = 64;       // K elements per stage (one 128-byte swizzle row)
static constexpr int STAGES = 6;
static constexpr int A_BYTES = BM * BK * 2;        // this CTA's x tile
static constexpr int B_BYTES = (BN / 2) * BK * 2;  // this CTA's half of the W tile
static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
static constexpr int THREADS = 192;
static constexpr int TMEM_COLS = 512;
// barriers: full[STAGES], empty[STAGES], tfull[2], tempty[2]
static constexpr int NUM_BARS = 2 * STAGES + 4;
// Stored softmax weights (kStore == 2) are taken relative to m_ref + this margin: bf16 then holds
// them for logits from 47 below to 128 above m_ref (the single pass uses the same reference).
static constexpr float STORED_WEIGHT_MARGIN = 40.f;
static constexpr int SMEM_BYTES = 1024 /*alignment slack*/ + STAGES * STAGE_BYTES + NUM_BARS * 8 + 64;
// kStore == 2: each epilogue warp stages 32 rows x 64 weights (4 KiB, the layout of a TMA box with
// 128-byte swizzle) in one of two buffers and stores it with one TMA instruction: whole 128-byte
// lines reach L2 instead of one 16-byte piece per thread and instruction.
static constexpr int ZSTAGE_OFF = STAGES * STAGE_BYTES + 1024;   // past the barriers, 1 KiB aligned
static constexpr int ZSTAGE_BYTES = 4 * 2 * 4096;
static constexpr int SMEM_BYTES_STORE = 1024 + ZSTAGE_OFF + ZSTAGE_BYTES;
static_assert(NUM_BARS * 8 + 64 <= 1024, "barriers overlap the staging buffers");
static_assert(SMEM_BYTES_STORE <= 227 * 1024, "shared memory");
}  // namespace fwd

// Folds 32 logits (one TMEM chunk of this thread's row) into the running record.
// `col0` = local vocabulary index of z[0]; `nvalid` = how many of the 32 are real columns.
struct RowState {
  float m, ml2, s, t2, tz;
  int idx;
};

template <bool kExclTarget = false>
__device__ __forceinline__ void fold_chunk(RowState& st, const uint32_t (&r)[32], int col0,
                                           int nvalid, int tgt_local) {
  float z[32];
#pragma unroll
  for (int j = 0; j < 32; ++j) z[j] = __uint_as_float(r[j]);
  if (nvalid < 32) {
#pragma unroll
    for (int j = 0; j < 32; ++j)
      if (j >= nvalid) z[j] = NEG_BIG;
  }
  float cm = z[0];
#pragma unroll
  for (int j = 1; j < 32; ++j) cm = fmaxf(cm, z[j]);
  if (cm > st.m) {
    // New row maximum: strict '>' keeps the earliest chunk; inside the chunk take the first hit.
    int jj = 31;
#pragma unroll
    for (int j = 30; j >= 0; --j)
      if (z[j] == cm) jj = j;
    st.idx = col0 + jj;
    const float dm2 = (st.m - cm) * LOG2E;  // <= 0, finite because NEG_BIG is finite
    const float sc = ex2_approx(dm2);
    st.t2 = sc * (st.t2 + st.s * dm2);
    st.s = sc * st.s;
    st.m = cm;
    st.ml2 = cm * LOG2E;
  }
  float cs0 = 0.f, cs1 = 0.f, ct0 = 0.f, ct1 = 0.f;
  const unsigned tl = static_cast<unsigned>(tgt_local - col0);
#pragma unroll
  for (int j = 0; j < 32; j += 2) {
    const float d0 = fmaf(z[j], LOG2E, -st.ml2);
    const float d1 = fmaf(z[j + 1], LOG2E, -st.ml2);
    float e0 = ex2_approx(d0);
    float e1 = ex2_approx(d1);
    if (kExclTarget) {   // the target's entry stays out of the sums
      if (static_cast<unsigned>(j) == tl) e0 = 0.f;
      if (static_cast<unsigned>(j + 1) == tl) e1 = 0.f;
    }
    cs0 += e0;
    cs1 += e1;
    ct0 = fmaf(e0, d0, ct0);
    ct1 = fmaf(e1, d1, ct1);
  }
  st.s += cs0 + cs1;
  st.t2 += ct0 + ct1;
  if (tl < 32u) {
#pragma unroll
    for (int j = 0; j < 32; ++j)
      if (static_cast<unsigned>(j) == tl) st.tz = z[j];
  }
}

template <int kFmt, int kStore = 0>  // kFmt: 0 = fp16, 1 = bf16; kStore: 0 none, 1 logits, 2 weights
__global__ void __launch_bounds__(fwd::THREADS, 1)
head_fwd_kernel(const __grid_constant__ CUtensorMap tmap_x,
                const __grid_constant__ CUtensorMap tmap_w,
                const __grid_constant__ CUtensorMap tmap_z,   // kStore == 2: zbuf, box {64, 32}
                const FwdParams p) {
  using namespace fwd;
  if (p.gate != nullptr && *p.gate == 0) return;   // guarded launch: not needed this time
  if (p.row_range != nullptr && p.row_range[1] <= p.row_range[0]) return;   // no rows to sweep
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;  // 128-byte swizzle wants 1024-byte tiles
  uint8_t* gen_base = smem_raw + (base - raw);
  const uint32_t bars = base + STAGES * STAGE_BYTES;
  auto full_bar = [&](int s) { return bars + 8u * s; };
  auto empty_bar = [&](int s) { return bars + 8u * (STAGES + s); };
  auto tfull_bar = [&](int a) { return bars + 8u * (2 * STAGES + a); };
  auto tempty_bar = [&](int a) { return bars + 8u * (2 * STAGES + 2 + a); };
  volatile uint32_t* tmem_slot =
      reinterpret_cast<volatile uint32_t*>(gen_base + STAGES * STAGE_BYTES + NUM_BARS * 8);
  volatile int* abort_flag =
      reinterpret_cast<volatile int*>(gen_base + STAGES * STAGE_BYTES + NUM_BARS * 8 + 8);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int kblocks = (p.h + BK - 1) / BK;
  const uint32_t c = cluster_ctarank();   // 0 = pair leader, 1 = peer
  const bool is_leader = (c == 0);
  const int pair_id = blockIdx.x >> 1;
  const int n_pairs = gridDim.x >> 1;
  // Rows and work split: from the host plan, or from the device row range.
  int row0 = 0, row_end = p.n, n_row_pairs = p.n_row_pairs, tiles_per_unit = p.tiles_per_unit;
  int n_splits = p.n_splits, pstride = p.n;
  if (p.row_range != nullptr) {
    row0 = p.row_range[0];
    row_end = min(p.row_range[1], p.n);
    const FwdSplit fs = fwd_split_rows(max(row_end - row0, 0), p.n_vtiles, n_pairs, p.part_cap);
    n_row_pairs = fs.n_row_pairs;
    tiles_per_unit = fs.tiles_per_unit;
    n_splits = fs.n_splits;
    pstride = fs.stride;
  }
  const int n_units = n_row_pairs * n_splits;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(tfull_bar(a), 1);
      mbar_init(tempty_bar(a), 8);  // one arrival per epilogue warp of both CTAs (leader's)
    }
    *abort_flag = 0;
    fence_barrier_init();
    fence_proxy_async();
    tma_prefetch_desc(&tmap_x);
    tma_prefetch_desc(&tmap_w);
  }
  if (warp == 1) {
    tmem_alloc_pair(smem_u32(const_cast<uint32_t*>(tmem_slot)), TMEM_COLS);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  cluster_arrive();  // the peer must see initialised barriers before any remote arrive
  cluster_wait();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------- TMA producer (whole warp, one lane issues) --------
    const bool elected = elect_one_sync();
    uint32_t stage = 0, phase = 0;
    bool ok = true;
    const uint32_t full_leader0 = mapa_shared(full_bar(0), 0);
    for (int u = pair_id; u < n_units && ok; u += n_pairs) {
      const int rt = 2 * (u % n_row_pairs) + static_cast<int>(c);
      const int sp = u / n_row_pairs;
      const int vt0 = sp * tiles_per_unit;
      const int vt1 = min(vt0 + tiles_per_unit, p.n_vtiles);
      for (int vt = vt0; vt < vt1 && ok; ++vt) {
        for (int kb = 0; kb < kblocks; ++kb) {
          ok = mbar_wait_warp<true>(empty_bar(stage), phase ^ 1u, abort_flag);
          if (!ok) break;
          if (elected) {
            const uint32_t sa = base + stage * STAGE_BYTES;
            // the leader's barrier counts the bytes of both CTAs
            if (is_leader) mbar_expect_tx(full_bar(stage), 2 * STAGE_BYTES);
            const uint32_t bar = full_leader0 + 8u * stage;
            tma_load_2d_pair(sa, &tmap_x, bar, kb * BK, row0 + rt * BM);
            tma_load_2d_pair(sa + A_BYTES, &tmap_w, bar, kb * BK,
                             vt * BN + static_cast<int>(c) * (BN / 2));
          }
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
    }
    if (!ok && elected) {
      *abort_flag = 1;
      atomicCAS(p.status, DEV_OK, DEV_TIMEOUT_PRODUCER);
    }
  } else if (warp == 1) {
    // ------------------- MMA issuer (pair leader only; whole warp, one lane issues) -----
    if (is_leader) {
      const bool elected = elect_one_sync();
      constexpr uint32_t idesc = make_idesc(kFmt, 2 * BM, BN, 0, 0);
      constexpr uint16_t kPairMask = 3;
      uint32_t stage = 0, phase = 0, acc = 0, aphase = 0;
      bool ok = true;
      for (int u = pair_id; u < n_units && ok; u += n_pairs) {
        const int sp = u / n_row_pairs;
        const int vt0 = sp * tiles_per_unit;
        const int vt1 = min(vt0 + tiles_per_unit, p.n_vtiles);
        for (int vt = vt0; vt < vt1 && ok; ++vt) {
          // both CTAs' epilogues must have drained this accumulator
          ok = mbar_wait_warp<true>(tempty_bar(acc), aphase ^ 1u, abort_flag);
          if (!ok) break;
          tc_fence_after();
          const uint32_t d_tmem = tmem_base + acc * BN;
          for (int kb = 0; kb < kblocks; ++kb) {
            ok = mbar_wait_warp<true>(full_bar(stage), phase, abort_flag);
            if (!ok) break;
            tc_fence_after();
            const uint32_t sa = base + stage * STAGE_BYTES;
            const uint64_t adesc = make_smem_desc(sa, 16, 1024);            // 128 rows of x
            const uint64_t bdesc = make_smem_desc(sa + A_BYTES, 16, 1024);  // 128 of 256 W rows
            if (elected) {
              // +32 bytes (16 K elements) inside the 128-byte swizzle row: +2 in >>4 units
              umma_f16_ss_pair(d_tmem, adesc, bdesc, idesc, kb != 0);
              umma_f16_ss_pair(d_tmem, adesc + 2u, bdesc + 2u, idesc, 1u);
              umma_f16_ss_pair(d_tmem, adesc + 4u, bdesc + 4u, idesc, 1u);
              umma_f16_ss_pair(d_tmem, adesc + 6u, bdesc + 6u, idesc, 1u);
              umma_commit_pair_mask(empty_bar(stage), kPairMask);
            }
            if (++stage == STAGES) {
              stage = 0;
              phase ^= 1u;
            }
          }
          if (ok && elected) umma_commit_pair_mask(tfull_bar(acc), kPairMask);
          acc ^= 1u;
          aphase ^= acc ^ 1u;  // flips when acc wraps back to 0
        }
      }
      if (!ok && elected) {
        *abort_flag = 1;
        atomicCAS(p.status, DEV_OK, DEV_TIMEOUT_MMA);
      }
    }
  } else {
    // ------------------------------- epilogue warps -----------------------------------
    const int quad = warp & 3;           // TMEM lane quadrant this warp may read
    const int row_in_tile = quad * 32 + lane;
    uint32_t acc = 0, aphase = 0;
    const uint32_t zstage = base + ZSTAGE_OFF + static_cast<uint32_t>(quad) * 8192u;
    uint32_t zpairs = 0;                 // chunk pairs this warp has stored (buffer = zpairs & 1)
    bool ok = true;
    const uint32_t tempty_leader0 = mapa_shared(tempty_bar(0), 0);
    for (int u = pair_id; u < n_units && ok; u += n_pairs) {
      const int rt = 2 * (u % n_row_pairs) + static_cast<int>(c);
      const int sp = u / n_row_pairs;
      const int vt0 = sp * tiles_per_unit;
      const int vt1 = min(vt0 + tiles_per_unit, p.n_vtiles);
      const int row = row0 + rt * BM + row_in_tile;
      int tgt_local = -1;
      float mref = 0.f;
      __half* zrow = nullptr;
      if (row < row_end) {
        const long long tg = p.target[row] - p.vocab_offset;
        if (tg >= 0 && tg < p.v) tgt_local = static_cast<int>(tg);
        if (kStore) {
          mref = p.m_ref[row];
          zrow = p.zbuf + static_cast<size_t>(row - row0) * p.zpitch;
        }
      }
      // kStore == 2: the warp stores its 32 rows together (rows past the end hold finite junk that
      // nothing reads)
      const bool zwarp = kStore == 2 && row0 + rt * BM + quad * 32 < row_end;
      RowState st;
      st.m = NEG_BIG;
      st.ml2 = NEG_BIG * LOG2E;
      st.s = 0.f;
      st.t2 = 0.f;
      st.tz = 0.f;
      st.idx = 0;
      for (int vt = vt0; vt < vt1 && ok; ++vt) {
        // warp-uniform outcome: tcgen05.ld below is a whole-warp instruction
        ok = mbar_wait_warp<true>(tfull_bar(acc), aphase, abort_flag);
        if (!ok) break;
        tc_fence_after();
        const uint32_t taddr = tmem_base + acc * BN + (static_cast<uint32_t>(quad * 32) << 16);
        const int v0 = vt * BN;
        const int tile_valid = min(BN, p.v - v0);
#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {
          uint32_t r[32];
          tmem_ld32(taddr + c * 32, r);
          tmem_ld_wait();
          const int nvalid = tile_valid - c * 32;
          if (kStore == 2 && zwarp) {
            // 32 softmax weights of this row relative to its reference maximum, as bf16
            uint32_t hw[16];
            const float mref2 = (mref + STORED_WEIGHT_MARGIN) * LOG2E;
#pragma unroll
            for (int e = 0; e < 16; ++e) {
              const __nv_bfloat162 hv = __floats2bfloat162_rn(
                  ex2_approx(fmaf(__uint_as_float(r[2 * e]), LOG2E, -mref2)),
                  ex2_approx(fmaf(__uint_as_float(r[2 * e + 1]), LOG2E, -mref2)));
              hw[e] = *reinterpret_cast<const uint32_t*>(&hv);
            }
            // entries that must read as zero: the target's (added in fp32 by the row finish) and
            // those past the end of the vocabulary
            const unsigned tl = static_cast<unsigned>(tgt_local - (v0 + c * 32));
            uint32_t keep = nvalid >= 32 ? 0xffffffffu : (nvalid <= 0 ? 0u : ((1u << nvalid) - 1u));
            if (tl < 32u) keep &= ~(1u << tl);
            if (keep != 0xffffffffu) {
#pragma unroll
              for (int e = 0; e < 16; ++e)
                hw[e] &= (((keep >> (2 * e)) & 1u) ? 0x0000ffffu : 0u) |
                         (((keep >> (2 * e + 1)) & 1u) ? 0xffff0000u : 0u);
            }
            // two chunks = one box of 64 weights x 32 rows: line = lane, 16-byte group XOR line & 7
            const uint32_t zb = zstage + (zpairs & 1u) * 4096u;
            if ((c & 1) == 0) {
              if (lane == 0) bulk_wait_group_read<1>();   // the store that last read this buffer
              __syncwarp();
            }
#pragma unroll
            for (int g = 0; g < 4; ++g)
              st_shared_v4(zb + static_cast<uint32_t>(lane * 128 + ((((c & 1) * 4 + g) ^ (lane & 7)) * 16)),
                           hw[4 * g], hw[4 * g + 1], hw[4 * g + 2], hw[4 * g + 3]);
            if (c & 1) {
              fence_proxy_async_shared();
              __syncwarp();
              if (lane == 0) {
                tma_store_2d(&tmap_z, zb, v0 + (c - 1) * 32, rt * BM + quad * 32);
                bulk_commit_group();
              }
              ++zpairs;
            }
          } else if (kStore == 1 && zrow != nullptr) {
            // 32 logits of this row, relative to its reference maximum and in units of ln 2, as 64
            // bytes of fp16 (the dHidden kernel's 2^x takes them as they are)
            uint4* dst = reinterpret_cast<uint4*>(zrow + v0 + c * 32);
#pragma unroll
            for (int g = 0; g < 4; ++g) {
              uint32_t hw[4];
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                const __half2 hv =
                    __floats2half2_rn((__uint_as_float(r[g * 8 + 2 * e]) - mref) * LOG2E,
                                      (__uint_as_float(r[g * 8 + 2 * e + 1]) - mref) * LOG2E);
                hw[e] = *reinterpret_cast<const uint32_t*>(&hv);
              }
              dst[g] = make_uint4(hw[0], hw[1], hw[2], hw[3]);
            }
          }
          if (nvalid > 0) fold_chunk<(kStore != 0)>(st, r, v0 + c * 32, nvalid, tgt_local);
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive_remote(tempty_leader0 + 8u * acc);
        acc ^= 1u;
        aphase ^= acc ^ 1u;  // flips when acc wraps back to 0
      }
      if (ok && row < row_end) {
        const size_t o = static_cast<size_t>(sp) * pstride + (row - row0);
        p.pm[o] = st.m;
        p.ps[o] = st.s;
        p.pt[o] = st.t2 * LN2;
        p.ptz[o] = st.tz;
        p.pidx[o] = st.idx;
      }
    }
    if (kStore == 2 && lane == 0) bulk_wait_group<0>();   // this warp's stores have landed
    if (!ok && lane == 0) {
      *abort_flag = 1;
      atomicCAS(p.status, DEV_OK, DEV_TIMEOUT_EPILOGUE);
    }
  }

  tc_fence_before();
  __syncthreads();
  cluster_arrive();  // nobody leaves while the peer may still arrive on this CTA's barriers
  cluster_wait();
  tc_fence_after();
  if (warp == 1) tmem_dealloc_pair(tmem_base, TMEM_COLS);
}

}  // namespace esep
