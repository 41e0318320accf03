// Router: gate logits with a fixed fp32 summation tree, softmax, top-k with renormalisation,
// and the routing lists the MoE GEMMs consume.
//
// Replaces the reference's route kernels (qk_route.cu:214 route_kernel, :496 route48_kernel, :972
// route16w_kernel) and their Triton twins (i8x_decode.py:226-289).  The reference multiplies bf16
// weights on mma.sync tensor cores; the target's router weight is fp32, so the gate is an fp32
// FMA kernel whose summation order is part of the contract:
//   p_s  = fma chain from 0 over k = 128 s .. 128 s + 127 (ascending), s = 0 .. H/128 - 1
//   logit = ((p_0 + p_1) + p_2) + ... ; bias added last.
// Sixteen-thread groups own one 128-deep slice each, so a 2048-deep dot product is 128 dependent
// FMAs long instead of 2048; the slices meet in shared memory and are added in slice order.
#include "common.cuh"
#include "host.h"

namespace b200 {

constexpr int RT_TOK = 16, RT_EXP = 16, RT_SLICE = 128, RT_THREADS = 256;

// grid (ceil(T/16), E/16, ceil(nslices/16)); block 256 = 16 slices x (4 x 4 thread tiles of 4 x 4 outputs)
__global__ void __launch_bounds__(RT_THREADS) router_logits_kernel(const bf16* __restrict__ x,
                                                                   const float* __restrict__ wr,
                                                                   const float* __restrict__ bias, int T, int H, int E,
                                                                   float* __restrict__ logits) {
  __shared__ float part[16][RT_TOK][RT_EXP + 1];
  const int tid = threadIdx.x;
  const int s_local = tid >> 4;            // slice owned inside a 16-slice pass
  const int ty = (tid >> 2) & 3, tx = tid & 3;
  const int t0 = blockIdx.x * RT_TOK + ty * 4, e0 = blockIdx.y * RT_EXP + tx * 4;
  const int nslices = H / RT_SLICE;
  const int ot = tid >> 4, oe = tid & 15;  // output owned in the combine phase
  float total = 0.f;
  for (int sbase = 0; sbase < nslices; sbase += 16) {
    const int s = sbase + s_local;
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
    if (s < nslices) {
      const bf16* xp[4];
      const float* wp[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int t = min(t0 + i, T - 1);  // rows past T are computed on a clamped row and dropped
        xp[i] = x + static_cast<size_t>(t) * H + s * RT_SLICE;
        wp[i] = wr + static_cast<size_t>(e0 + i) * H + s * RT_SLICE;
      }
#pragma unroll 2
      for (int k = 0; k < RT_SLICE; k += 8) {
        float xv[4][8], wv[4][8];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const uint4 xr = __ldg(reinterpret_cast<const uint4*>(xp[i] + k));
          xv[i][0] = bf_lo(xr.x); xv[i][1] = bf_hi(xr.x); xv[i][2] = bf_lo(xr.y); xv[i][3] = bf_hi(xr.y);
          xv[i][4] = bf_lo(xr.z); xv[i][5] = bf_hi(xr.z); xv[i][6] = bf_lo(xr.w); xv[i][7] = bf_hi(xr.w);
          const float4 w0 = __ldg(reinterpret_cast<const float4*>(wp[i] + k));
          const float4 w1 = __ldg(reinterpret_cast<const float4*>(wp[i] + k + 4));
          wv[i][0] = w0.x; wv[i][1] = w0.y; wv[i][2] = w0.z; wv[i][3] = w0.w;
          wv[i][4] = w1.x; wv[i][5] = w1.y; wv[i][6] = w1.z; wv[i][7] = w1.w;
        }
#pragma unroll
        for (int kk = 0; kk < 8; ++kk)
#pragma unroll
          for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) acc[i][j] = __fmaf_rn(xv[i][kk], wv[j][kk], acc[i][j]);
      }
    }
    __syncthreads();  // previous pass's partials have been consumed
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) part[s_local][ty * 4 + i][tx * 4 + j] = acc[i][j];
    __syncthreads();
    const int lim = min(16, nslices - sbase);
    for (int q = 0; q < lim; ++q) {
      const float pv = part[q][ot][oe];
      total = (sbase + q == 0) ? pv : __fadd_rn(total, pv);
    }
  }
  const int t = blockIdx.x * RT_TOK + ot, e = blockIdx.y * RT_EXP + oe;
  if (t < T) {
    if (bias) total = __fadd_rn(total, __ldg(bias + e));
    logits[static_cast<size_t>(t) * E + e] = total;
  }
}

// Sortable key: larger logit first, then smaller expert id; -0 == +0; NaN ranks below everything
// (the reference's 24-bit key has the same order: qk_route.cu:71-75,142).
__device__ __forceinline__ unsigned long long topk_key(float v, int id) {
  uint32_t u;
  if (v != v) {
    u = 0u;
  } else {
    v += 0.f;  // -0 -> +0
    u = __float_as_uint(v);
    u = (u & 0x80000000u) ? ~u : (u | 0x80000000u);
    if (u == 0u) u = 1u;
  }
  return (static_cast<unsigned long long>(u) << 32) | static_cast<uint32_t>(0xffffffffu - static_cast<uint32_t>(id));
}

// one warp per token; lane l holds experts l, l + 32, ...
template <int PER_LANE>
__global__ void __launch_bounds__(256) router_topk_kernel(const float* __restrict__ logits, int T, int E, int K,
                                                          int round_bf16, int32_t* __restrict__ ids,
                                                          float* __restrict__ wts) {
  const int lane = threadIdx.x & 31;
  const int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (t >= T) return;
  float xv[PER_LANE];
  unsigned long long key[PER_LANE];
  float mx = -INFINITY;
#pragma unroll
  for (int j = 0; j < PER_LANE; ++j) {
    const int e = lane + 32 * j;
    float v = e < E ? logits[static_cast<size_t>(t) * E + e] : -INFINITY;
    if (round_bf16) v = rbf(v);
    xv[j] = v;
    key[j] = e < E ? topk_key(v, e) : 0ull;
    if (v == v) mx = fmaxf(mx, v);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(FULL_MASK, mx, o));
  float sum = 0.f;
#pragma unroll
  for (int j = 0; j < PER_LANE; ++j) {
    const float v = xv[j];
    const float ex = (v == v && lane + 32 * j < E) ? expf(v - mx) : 0.f;
    xv[j] = ex;
    sum += ex;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(FULL_MASK, sum, o);
  float my_w = 0.f;   // lane k keeps the k-th pick
  int my_id = 0;
  float tot = 0.f;
  for (int k = 0; k < K; ++k) {
    unsigned long long best = 0ull;
    int bj = 0;
#pragma unroll
    for (int j = 0; j < PER_LANE; ++j)
      if (key[j] > best) {
        best = key[j];
        bj = j;
      }
    unsigned long long win = best;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const unsigned long long other = __shfl_xor_sync(FULL_MASK, win, o);
      win = other > win ? other : win;
    }
    const int id = static_cast<int>(0xffffffffu - static_cast<uint32_t>(win & 0xffffffffull));
    const int owner = id & 31;
    float pr = 0.f;
    if (lane == owner) {
#pragma unroll
      for (int j = 0; j < PER_LANE; ++j)
        if (j == bj) {
          pr = __fdiv_rn(xv[j], sum);
          key[j] = 0ull;
        }
    }
    pr = __shfl_sync(FULL_MASK, pr, owner);
    tot = __fadd_rn(tot, pr);
    if (lane == k) {
      my_w = pr;
      my_id = id;
    }
  }
  const float den = tot > 0.f ? tot : 1.f;
  if (lane < K) {
    ids[static_cast<size_t>(t) * K + lane] = my_id;
    wts[static_cast<size_t>(t) * K + lane] = __fdiv_rn(my_w, den);
  }
}

// ---- routing lists ---------------------------------------------------------------------------------
// One CTA.  Warp 0 ranks the routed pairs in slot order (stable inside an expert) with match.any;
// the whole CTA then scatters rows and writes the block list.
constexpr int LISTS_THREADS = 1024, LISTS_MAX_E = 1024;

__global__ void __launch_bounds__(LISTS_THREADS) moe_lists_kernel(const int32_t* __restrict__ ids,
                                                                  const float* __restrict__ wts,
                                                                  const int64_t* __restrict__ pos, int T, int K,
                                                                  int e_lo, int E_local, int block_rows,
                                                                  int with_shared, int max_blocks, MoeLists L) {
  __shared__ int cnt[LISTS_MAX_E + 1];
  __shared__ int off[LISTS_MAX_E + 2];
  __shared__ int bstart[LISTS_MAX_E + 2];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int P = T * K;
  for (int e = tid; e <= E_local; e += LISTS_THREADS) cnt[e] = 0;
  for (int r = tid; r < T * (K + 1); r += LISTS_THREADS) {
    L.slot_of_row[r] = -1;
    L.wt_of_row[r] = 0.f;
  }
  __syncthreads();
  if (warp == 0) {
    for (int p0 = 0; p0 < P; p0 += 32) {
      const int p = p0 + lane;
      int le = -1;
      if (p < P) {
        const int e = ids[p] - e_lo;
        const bool ok = (pos == nullptr) || (pos[p / K] != 0);
        if (ok && e >= 0 && e < E_local) le = e;
      }
      const unsigned same = __match_any_sync(FULL_MASK, le);
      const int before = __popc(same & ((1u << lane) - 1u));
      int base = 0;
      if (le >= 0) base = cnt[le];
      __syncwarp();
      if (le >= 0 && before == 0) cnt[le] = base + __popc(same);
      __syncwarp();
      if (p < P) L.row_of_pair[p] = le >= 0 ? base + before : -1;  // rank for now
    }
  }
  __syncthreads();
  if (tid == 0) {
    int run = 0, blocks = 0;
    for (int e = 0; e < E_local; ++e) {
      off[e] = run;
      bstart[e] = blocks;
      run += cnt[e];
      blocks += (cnt[e] + block_rows - 1) / block_rows;
    }
    off[E_local] = P;  // the shared expert's rows start after the routed region
    cnt[E_local] = with_shared ? T : 0;
    bstart[E_local] = blocks;
    blocks += (cnt[E_local] + block_rows - 1) / block_rows;
    off[E_local + 1] = P + cnt[E_local];
    bstart[E_local + 1] = blocks;
    L.nblocks[0] = blocks <= max_blocks ? blocks : 0;
  }
  __syncthreads();
  for (int e = tid; e <= E_local; e += LISTS_THREADS) L.counts[e] = cnt[e];
  for (int e = tid; e <= E_local + 1; e += LISTS_THREADS) L.offsets[e] = off[e];
  for (int p = tid; p < P; p += LISTS_THREADS) {
    const int rank = L.row_of_pair[p];
    if (rank >= 0) {
      const int row = off[ids[p] - e_lo] + rank;
      L.row_of_pair[p] = row;
      L.slot_of_row[row] = p;
      L.wt_of_row[row] = wts[p];
    }
  }
  if (with_shared)
    for (int t = tid; t < T; t += LISTS_THREADS) {
      const bool ok = (pos == nullptr) || (pos[t] != 0);
      L.slot_of_row[P + t] = ok ? P + t : -1;
      L.wt_of_row[P + t] = 1.f;
    }
  if (bstart[E_local + 1] <= max_blocks)
    for (int e = tid; e <= E_local; e += LISTS_THREADS) {
      const int c = cnt[e];
      int b = bstart[e];
      for (int r0 = 0; r0 < c; r0 += block_rows, ++b) {
        L.blk_expert[b] = e;
        L.blk_row0[b] = off[e] + r0;
        L.blk_rows[b] = min(block_rows, c - r0);
      }
    }
}

}  // namespace b200

using namespace b200;

extern "C" int b200_router(const void* x, const float* wr, const float* bias, int T, int H, int E, int K, int flags,
                           float* logits, int32_t* ids, float* wts, void* stream) {
  if (!x || !wr || !logits || !ids || !wts) return fail(B200_E_ARG, "b200_router: null pointer");
  if (T < 0 || H <= 0 || H % RT_SLICE || E <= 0 || E % 32 || E > 1024 || K <= 0 || K > 32 || K > E)
    return fail(B200_E_ARG, "b200_router: need H %% 128 == 0, E %% 32 == 0, E <= 1024, 1 <= K <= 32 (T=%d H=%d E=%d K=%d)",
                T, H, E, K);
  if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(wr)) & 15)
    return fail(B200_E_ALIGN, "b200_router: x and wr must be 16-byte aligned");
  if (T == 0) return 0;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  dim3 grid((T + RT_TOK - 1) / RT_TOK, E / RT_EXP);
  router_logits_kernel<<<grid, RT_THREADS, 0, st>>>(static_cast<const bf16*>(x), wr, bias, T, H, E, logits);
  const int per_lane = (E + 31) / 32;
  dim3 g2((T + 7) / 8);
  const int rb = flags & 1;
  if (per_lane <= 8)
    router_topk_kernel<8><<<g2, 256, 0, st>>>(logits, T, E, K, rb, ids, wts);
  else if (per_lane <= 16)
    router_topk_kernel<16><<<g2, 256, 0, st>>>(logits, T, E, K, rb, ids, wts);
  else
    router_topk_kernel<32><<<g2, 256, 0, st>>>(logits, T, E, K, rb, ids, wts);
  return launch_status("b200_router");
}

extern "C" int b200_moe_max_blocks(int T, int K, int E_local, int block_rows) {
  if (T < 0 || K <= 0 || E_local < 0 || block_rows <= 0) return B200_E_ARG;
  // every local expert may end with one partial block; the shared expert adds ceil(T / block_rows)
  return E_local + (T * K) / block_rows + (T + block_rows - 1) / block_rows + 1;
}

extern "C" int b200_moe_build_lists(const int32_t* ids, const float* wts, const int64_t* pos, int T, int K, int e_lo,
                                    int E_local, int block_rows, int with_shared, const b200_moe_lists* lists,
                                    void* stream) {
  if (!ids || !wts || !lists || !lists->counts || !lists->offsets || !lists->row_of_pair || !lists->slot_of_row ||
      !lists->wt_of_row || !lists->blk_expert || !lists->blk_row0 || !lists->blk_rows || !lists->nblocks)
    return fail(B200_E_ARG, "b200_moe_build_lists: null pointer");
  if (T <= 0 || K <= 0 || E_local <= 0 || E_local > LISTS_MAX_E || e_lo < 0 || block_rows < 16 || block_rows > 128 ||
      block_rows % 16)
    return fail(B200_E_ARG, "b200_moe_build_lists: bad shape (T=%d K=%d E_local=%d block_rows=%d)", T, K, E_local,
                block_rows);
  MoeLists L{lists->counts,     lists->offsets,  lists->row_of_pair, lists->slot_of_row, lists->wt_of_row,
             lists->blk_expert, lists->blk_row0, lists->blk_rows,    lists->nblocks};
  moe_lists_kernel<<<1, LISTS_THREADS, 0, static_cast<cudaStream_t>(stream)>>>(
      ids, wts, pos, T, K, e_lo, E_local, block_rows, with_shared, b200_moe_max_blocks(T, K, E_local, block_rows), L);
  return launch_status("b200_moe_build_lists");
}
