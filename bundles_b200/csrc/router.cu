// Router: gate logits with a fixed fp32 summation tree, softmax, top-k with renormalisation,
// and the routing lists the MoE GEMMs consume.
//
// Replaces the reference's route kernels (qk_route.cu:214 route_kernel, :496 route48_kernel, :972
// route16w_kernel) and their Triton twins (i8x_decode.py:226-289).  The reference multiplies bf16
// weights on mma.sync tensor cores; the target's router weight is fp32, so the gate is an fp32
// FMA kernel whose summation order is part of the contract:
//   p_s  = fma chain from 0 over k = 128 s .. 128 s + 127 (ascending), s = 0 .. H/128 - 1
//   logit = ((p_0 + p_1) + p_2) + ... ; bias added last.
// Each 128-deep slice is computed by its own CTAs (a 2048-deep dot product is then 128 dependent
// FMAs long and 16 times more parallel); the top-k kernel adds the slice partials in slice order.
#include "common.cuh"
#include "host.h"

#include <mutex>

namespace b200 {

B200_DEFINE_WAIT_BUDGET_SETTER(set_wait_budget_router)

constexpr int RT_EXP = 64, RT_SLICE = 128, RT_THREADS = 256, RT_PITCH = RT_SLICE + 4;
constexpr int RT_XPITCH = RT_SLICE + 8;  // bf16 elements per staged x row (272 bytes: 16-byte aligned, rows on different banks)
constexpr int RT_WBUF = RT_EXP * RT_PITCH * 4;
template <int TOK>
struct RtCfg {  // token-tile height: 64 (4 tokens per thread) up to 64 tokens, 128 (8 per thread) beyond
  static constexpr int XRAW = TOK * RT_XPITCH * 2, XS = TOK * RT_PITCH * 4;
  static constexpr int SMEM = 2 * RT_WBUF + 2 * XRAW + XS;
};

__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gsrc) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(smem_dst)), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// A unit of work is a TOK-token x 64-expert tile of ONE 128-deep k slice.  Persistent CTAs (one per SM) take
// units b, b + grid, ...: the next unit's operand tiles stream into shared memory with cp.async while the
// current one is computed, so the FMA pipe never waits for a staging round trip and the last wave is not
// a whole wave.  Both tiles are read as fp32 from shared memory (rows padded to 132 floats so 16-byte
// reads of consecutive rows hit different banks; x is converted from its staged bf16 copy first); each
// thread owns TOK/16 tokens x 4 experts and runs their fma chains over the slice in ascending k (with 8 tokens
// per thread there are 12 shared-memory reads per 128 FMAs instead of 8 per 64).  Slice partials go to
// `part[s][t][e]`; the top-k kernel adds them in slice order.
template <int RT_TOK>
__global__ void __launch_bounds__(RT_THREADS, 1) router_partials_kernel(const bf16* __restrict__ x,
                                                                        const float* __restrict__ wr, int T, int H,
                                                                        int E, float* __restrict__ part) {
  extern __shared__ __align__(16) uint8_t rt_smem[];
  auto wbuf = [&](int b) { return reinterpret_cast<float*>(rt_smem + b * RT_WBUF); };
  constexpr int RT_XRAW = RtCfg<RT_TOK>::XRAW, TI = RT_TOK / 16;
  auto xraw = [&](int b) { return reinterpret_cast<bf16*>(rt_smem + 2 * RT_WBUF + b * RT_XRAW); };
  float* xs = reinterpret_cast<float*>(rt_smem + 2 * RT_WBUF + 2 * RT_XRAW);
  const int tid = threadIdx.x;
  const int ttiles = (T + RT_TOK - 1) / RT_TOK, etiles = E / RT_EXP, nslices = H / RT_SLICE;
  const int nunits = ttiles * etiles * nslices;
  pdl_wait();
  pdl_launch();
  // unit -> (slice, token tile, expert tile), expert tile fastest
  auto issue = [&](int u, int buf) {
    const int et = u % etiles, tt = (u / etiles) % ttiles, s = u / (etiles * ttiles);
    const int t0 = tt * RT_TOK, e0 = et * RT_EXP;
    for (int i = tid; i < RT_EXP * (RT_SLICE / 4); i += RT_THREADS) {
      const int r = i >> 5, c = (i & 31) * 4;
      cp_async16(wbuf(buf) + r * RT_PITCH + c, wr + static_cast<size_t>(e0 + r) * H + s * RT_SLICE + c);
    }
    for (int i = tid; i < RT_TOK * (RT_SLICE / 8); i += RT_THREADS) {
      const int r = i >> 4, c = (i & 15) * 8;
      const int t = min(t0 + r, T - 1);  // rows past T repeat the last row and are dropped at the store
      cp_async16(xraw(buf) + r * RT_XPITCH + c, x + static_cast<size_t>(t) * H + s * RT_SLICE + c);
    }
    cp_async_commit();
  };
  int buf = 0;
  if (static_cast<int>(blockIdx.x) < nunits) issue(blockIdx.x, 0);
  for (int u = blockIdx.x; u < nunits; u += gridDim.x, buf ^= 1) {
    const int next = u + gridDim.x;
    if (next < nunits) {
      issue(next, buf ^ 1);
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();  // this unit's tiles have landed (every thread waited for its own copies)
    for (int i = tid; i < RT_TOK * (RT_SLICE / 8); i += RT_THREADS) {
      const int r = i >> 4, c = (i & 15) * 8;
      const uint4 v = *reinterpret_cast<const uint4*>(xraw(buf) + r * RT_XPITCH + c);
      float* d = xs + r * RT_PITCH + c;
      *reinterpret_cast<float4*>(d) = make_float4(bf_lo(v.x), bf_hi(v.x), bf_lo(v.y), bf_hi(v.y));
      *reinterpret_cast<float4*>(d + 4) = make_float4(bf_lo(v.z), bf_hi(v.z), bf_lo(v.w), bf_hi(v.w));
    }
    __syncthreads();
    const float* ws = wbuf(buf);
    const int ty = tid >> 4, tx = tid & 15;  // tokens ty + 16 i, experts tx + 16 j
    float acc[TI][4];
#pragma unroll
    for (int i = 0; i < TI; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
#pragma unroll 4
    for (int k = 0; k < RT_SLICE; k += 4) {
      float4 xv[TI], wv[4];
#pragma unroll
      for (int i = 0; i < TI; ++i) xv[i] = *reinterpret_cast<const float4*>(xs + (ty + 16 * i) * RT_PITCH + k);
#pragma unroll
      for (int j = 0; j < 4; ++j) wv[j] = *reinterpret_cast<const float4*>(ws + (tx + 16 * j) * RT_PITCH + k);
#pragma unroll
      for (int i = 0; i < TI; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          acc[i][j] = __fmaf_rn(xv[i].x, wv[j].x, acc[i][j]);
          acc[i][j] = __fmaf_rn(xv[i].y, wv[j].y, acc[i][j]);
          acc[i][j] = __fmaf_rn(xv[i].z, wv[j].z, acc[i][j]);
          acc[i][j] = __fmaf_rn(xv[i].w, wv[j].w, acc[i][j]);
        }
    }
    const int et = u % etiles, tt = (u / etiles) % ttiles, s = u / (etiles * ttiles);
    const int t0 = tt * RT_TOK, e0 = et * RT_EXP;
#pragma unroll
    for (int i = 0; i < TI; ++i) {
      const int t = t0 + ty + 16 * i;
      if (t < T)
#pragma unroll
        for (int j = 0; j < 4; ++j)
          part[(static_cast<size_t>(s) * T + t) * E + e0 + tx + 16 * j] = acc[i][j];
    }
    __syncthreads();  // xs and this unit's buffers are free for the copies issued in the next iteration
  }
}

// Sortable 32-bit key of a logit: larger first; -0 == +0; NaN ranks below every number (key 1);
// key 0 marks an entry that is absent or already picked.  Ties between equal keys go to the
// smaller expert id (the reference's order: qk_route.cu:71-75,142).
__device__ __forceinline__ uint32_t topk_key(float v) {
  if (v != v) return 1u;
  v += 0.f;  // -0 -> +0
  uint32_t u = __float_as_uint(v);
  u = (u & 0x80000000u) ? ~u : (u | 0x80000000u);
  return u < 2u ? 2u : u;
}
__device__ __forceinline__ float topk_unkey(uint32_t u) {
  return __uint_as_float((u & 0x80000000u) ? (u & 0x7fffffffu) : ~u);
}

// One CTA of four warps per token.  Warp w owns experts [w * E/4, (w+1) * E/4), lane l holds experts
// base + l + 32 j.  Each lane adds its experts' slice partials in slice order (+ bias); every load of
// the token is in flight at once.  Each warp then takes its own top K with two redux instructions per
// pick (warp max of the value key, warp min of the id among the lanes that hold it); warp 0 merges the
// 4 K candidates the same way.  Softmax statistics go through shared memory.
constexpr int TK_WARPS = 4;
template <int PL>  // experts per lane: ceil(E / 128)
__global__ void __launch_bounds__(128) router_topk_kernel(const float* __restrict__ part, int nslices,
                                                          const float* __restrict__ bias, int T, int E, int K,
                                                          int round_bf16, float* __restrict__ logits,
                                                          int32_t* __restrict__ ids, float* __restrict__ wts) {
  __shared__ float s_max[TK_WARPS], s_sum[TK_WARPS];
  __shared__ uint32_t c_key[TK_WARPS * 32];
  __shared__ int c_id[TK_WARPS * 32];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int t = blockIdx.x;
  pdl_wait();
  pdl_launch();
  const int EW = E / TK_WARPS;  // experts of this warp; entry j of lane l exists when l + 32 j < EW
  const int ebase = warp * EW;
  float xv[PL];
#pragma unroll
  for (int j = 0; j < PL; ++j) xv[j] = 0.f;
  {
    // slice partials: groups of 8 slices, all loads of a group issued before its adds
    for (int s0 = 0; s0 < nslices; s0 += 8) {
      float pv[8][PL];
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const float* pr = part + (static_cast<size_t>(min(s0 + u, nslices - 1)) * T + t) * E + ebase + lane;
#pragma unroll
        for (int j = 0; j < PL; ++j) pv[u][j] = (lane + 32 * j < EW) ? __ldg(pr + 32 * j) : 0.f;
      }
#pragma unroll
      for (int u = 0; u < 8; ++u)
        if (s0 + u < nslices) {
#pragma unroll
          for (int j = 0; j < PL; ++j) xv[j] = (s0 + u == 0) ? pv[u][j] : __fadd_rn(xv[j], pv[u][j]);
        }
    }
  }
  uint32_t key[PL];
  float mx = -INFINITY;
#pragma unroll
  for (int j = 0; j < PL; ++j) {
    const int e = ebase + lane + 32 * j;
    float v = xv[j];
    if (lane + 32 * j < EW) {
      if (bias) v = __fadd_rn(v, __ldg(bias + e));
      if (logits) logits[static_cast<size_t>(t) * E + e] = v;
      if (round_bf16) v = rbf(v);
      key[j] = topk_key(v);
      if (v == v) mx = fmaxf(mx, v + 0.f);
    } else {
      key[j] = 0u;
      v = __int_as_float(0x7fc00000);  // absent: contributes nothing to the softmax sum
    }
    xv[j] = v;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(FULL_MASK, mx, o));
  if (lane == 0) s_max[warp] = mx;
  __syncthreads();
  mx = fmaxf(fmaxf(s_max[0], s_max[1]), fmaxf(s_max[2], s_max[3]));
  float sum = 0.f;
#pragma unroll
  for (int j = 0; j < PL; ++j) {
    const float v = xv[j];
    sum += (v == v) ? expf((v + 0.f) - mx) : 0.f;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(FULL_MASK, sum, o);
  if (lane == 0) s_sum[warp] = sum;
  // this warp's top K (K <= 32): lane k keeps the k-th pick
  uint32_t bk = 0u;
  int bj = 0;
#pragma unroll
  for (int j = 0; j < PL; ++j)
    if (key[j] > bk) {
      bk = key[j];
      bj = j;
    }
  uint32_t my_key = 0u;
  int my_id = 0x7fffffff;
  const int Kw = min(K, E / TK_WARPS);
  for (int k = 0; k < Kw; ++k) {
    const uint32_t m = __reduce_max_sync(FULL_MASK, bk);
    const uint32_t cand = (bk == m) ? static_cast<uint32_t>(ebase + lane + 32 * bj) : 0x7fffffffu;
    const int id = static_cast<int>(__reduce_min_sync(FULL_MASK, cand));
    if (lane == k) {
      my_key = m;
      my_id = id;
    }
    if (lane == ((id - ebase) & 31)) {  // the owner drops the pick and rescans its entries
      const int dead = (id - ebase) >> 5;
      bk = 0u;
      bj = 0;
#pragma unroll
      for (int j = 0; j < PL; ++j) {
        if (j == dead) key[j] = 0u;
        if (key[j] > bk) {
          bk = key[j];
          bj = j;
        }
      }
    }
  }
  c_key[warp * 32 + lane] = my_key;  // lanes >= Kw hold key 0 (absent)
  c_id[warp * 32 + lane] = my_id;
  __syncthreads();
  if (warp != 0) return;
  sum = (s_sum[0] + s_sum[1]) + (s_sum[2] + s_sum[3]);
  // merge: lane l holds candidate l of every warp; pick by larger key, then smaller id
  uint32_t ck[TK_WARPS];
  int ci[TK_WARPS];
#pragma unroll
  for (int w = 0; w < TK_WARPS; ++w) {
    ck[w] = c_key[w * 32 + lane];
    ci[w] = c_id[w * 32 + lane];
  }
  auto rescan = [&](uint32_t& best_k, int& best_i) {
    best_k = 0u;
    best_i = 0x7fffffff;
#pragma unroll
    for (int w = 0; w < TK_WARPS; ++w)
      if (ck[w] > best_k || (ck[w] == best_k && ck[w] != 0u && ci[w] < best_i)) {
        best_k = ck[w];
        best_i = ci[w];
      }
  };
  int bi;
  rescan(bk, bi);
  float my_w = 0.f, tot = 0.f;
  int out_id = 0;
  for (int k = 0; k < K; ++k) {
    const uint32_t m = __reduce_max_sync(FULL_MASK, bk);
    const int id = static_cast<int>(__reduce_min_sync(FULL_MASK, (bk == m) ? static_cast<uint32_t>(bi) : 0x7fffffffu));
    const float pr = m <= 1u ? 0.f : __fdiv_rn(expf(topk_unkey(m) - mx), sum);
    tot = __fadd_rn(tot, pr);
    if (lane == k) {
      my_w = pr;
      out_id = id;
    }
    if (bk == m && bi == id) {  // exactly one lane holds this (key, id)
#pragma unroll
      for (int w = 0; w < TK_WARPS; ++w)
        if (ck[w] == m && ci[w] == id) ck[w] = 0u;
      rescan(bk, bi);
    }
  }
  const float den = tot > 0.f ? tot : 1.f;
  if (lane < K) {
    ids[static_cast<size_t>(t) * K + lane] = out_id;
    wts[static_cast<size_t>(t) * K + lane] = __fdiv_rn(my_w, den);
  }
}

// ---- routing lists ---------------------------------------------------------------------------------
// One CTA of 32 warps.  The local expert of every routed pair is staged in shared memory; warp w
// ranks its contiguous segment of pairs with match.any against its own counters, a per-expert scan
// over the 32 warps turns those into stable ranks (ascending slot order inside an expert), then
// rows are scattered and the block list is written.
constexpr int LISTS_THREADS = 1024, LISTS_WARPS = 32, LISTS_MAX_E = 1024;

__global__ void __launch_bounds__(LISTS_THREADS) moe_lists_kernel(const int32_t* __restrict__ ids,
                                                                  const float* __restrict__ wts,
                                                                  const int64_t* __restrict__ pos, int T, int K,
                                                                  int e_lo, int E_local, int block_rows,
                                                                  int shared_lo, int shared_n, int max_blocks, MoeLists L) {
  extern __shared__ int lists_smem[];
  pdl_wait();
  pdl_launch();
  const int P = T * K;
  const int E1 = E_local + 1;
  int* cnt = lists_smem;                   // [E1]   rows per expert
  int* off = cnt + E1;                     // [E1+1] first row per expert
  int* bstart = off + E1 + 1;              // [E1+1] first block per expert
  int* wsum = bstart + E1 + 1;             // [128]  scan scratch
  uint16_t* cntw = reinterpret_cast<uint16_t*>(wsum + 128);        // [32][E1] per-warp counters -> bases
  int16_t* sid = reinterpret_cast<int16_t*>(cntw + LISTS_WARPS * E1);  // [P] local expert or -1
  uint16_t* srank = reinterpret_cast<uint16_t*>(sid + P);              // [P] rank inside the warp segment
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;

  for (int i = tid; i < LISTS_WARPS * E1; i += LISTS_THREADS) cntw[i] = 0;
  for (int p = tid; p < P; p += LISTS_THREADS) {
    const int e = ids[p] - e_lo;
    const bool ok = (pos == nullptr) || (pos[p / K] != 0);
    sid[p] = (ok && e >= 0 && e < E_local) ? static_cast<int16_t>(e) : static_cast<int16_t>(-1);
  }
  for (int r = tid; r < T * (K + 1); r += LISTS_THREADS) {
    L.slot_of_row[r] = -1;
    L.wt_of_row[r] = 0.f;
  }
  __syncthreads();
  const int seg = ((P + LISTS_WARPS - 1) / LISTS_WARPS + 31) & ~31;
  {
    uint16_t* mine = cntw + warp * E1;
    const int p_end = min(P, (warp + 1) * seg);
    for (int p0 = warp * seg; p0 < p_end; p0 += 32) {
      const int p = p0 + lane;
      const int le = p < p_end ? sid[p] : -1;
      const unsigned same = __match_any_sync(FULL_MASK, le);
      const int before = __popc(same & ((1u << lane) - 1u));
      int base = 0;
      if (le >= 0) base = mine[le];
      __syncwarp();
      if (le >= 0 && before == 0) mine[le] = static_cast<uint16_t>(base + __popc(same));
      __syncwarp();
      if (p < p_end) srank[p] = static_cast<uint16_t>(base + before);
    }
  }
  __syncthreads();
  // per expert: exclusive scan of the warp counters -> base of each warp's segment; total -> cnt
  int c = 0;
  if (tid < E1) {
    if (tid < E_local) {
      int run = 0;
      for (int w = 0; w < LISTS_WARPS; ++w) {
        const int v = cntw[w * E1 + tid];
        cntw[w * E1 + tid] = static_cast<uint16_t>(run);
        run += v;
      }
      c = run;
    } else {
      c = shared_n;  // tokens [shared_lo, shared_lo + shared_n) get a shared-expert row
    }
    cnt[tid] = c;
  }
  // Blocks are listed heaviest first: all full blocks, then the partial blocks by quarter of the block size
  // (3/4 and more, 1/2, 1/4, less), each class in expert order.  The GEMMs deal tiles to their CTAs round-robin, so every CTA gets its share of
  // the expensive tiles instead of whatever the expert order happens to give it.
  // (Lists with smaller blocks feed the fp8 GEMMs, whose CTAs take contiguous tile ranges: those keep expert order.)
  const bool heavy_first = block_rows == 128;
  const int nfull = heavy_first ? c / block_rows : (c + block_rows - 1) / block_rows;
  const int tail = heavy_first ? c - nfull * block_rows : 0;
  const int pcls = tail == 0 ? -1 : 3 - min(3, (4 * tail) / block_rows);  // 0: >= 3/4 of a block ... 3: < 1/4
  const unsigned long long pone = pcls < 0 ? 0ull : 1ull << (16 * pcls);
  // block-wide exclusive scans of (rows of routed experts, blocks by class) over experts: the four partial classes
  // share one 64-bit word (16 bits each: at most one block per expert and class)
  int rows_incl = (tid < E_local) ? c : 0, blks_incl = nfull;
  unsigned long long part_incl = pone;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int a = __shfl_up_sync(FULL_MASK, rows_incl, o), b2 = __shfl_up_sync(FULL_MASK, blks_incl, o);
    const unsigned long long p2 = __shfl_up_sync(FULL_MASK, part_incl, o);
    if (lane >= o) {
      rows_incl += a;
      blks_incl += b2;
      part_incl += p2;
    }
  }
  if (lane == 31) {
    wsum[warp] = rows_incl;
    wsum[32 + warp] = blks_incl;
    wsum[64 + 2 * warp] = static_cast<int>(part_incl & 0xffffffffull);
    wsum[65 + 2 * warp] = static_cast<int>(part_incl >> 32);
  }
  __syncthreads();
  if (warp == 0) {
    int a = wsum[lane], b2 = wsum[32 + lane];
    unsigned long long p3 = static_cast<unsigned int>(wsum[64 + 2 * lane]) |
                            (static_cast<unsigned long long>(static_cast<unsigned int>(wsum[65 + 2 * lane])) << 32);
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int a2 = __shfl_up_sync(FULL_MASK, a, o), b3 = __shfl_up_sync(FULL_MASK, b2, o);
      const unsigned long long p4 = __shfl_up_sync(FULL_MASK, p3, o);
      if (lane >= o) {
        a += a2;
        b2 += b3;
        p3 += p4;
      }
    }
    wsum[lane] = a;
    wsum[32 + lane] = b2;
    wsum[64 + 2 * lane] = static_cast<int>(p3 & 0xffffffffull);
    wsum[65 + 2 * lane] = static_cast<int>(p3 >> 32);
  }
  __syncthreads();
  const int rows_excl = rows_incl - ((tid < E_local) ? c : 0) + (warp ? wsum[warp - 1] : 0);
  const int full_excl = blks_incl - nfull + (warp ? wsum[32 + warp - 1] : 0);
  auto wsum64 = [&](int w) {
    return static_cast<unsigned int>(wsum[64 + 2 * w]) |
           (static_cast<unsigned long long>(static_cast<unsigned int>(wsum[65 + 2 * w])) << 32);
  };
  const unsigned long long part_excl = part_incl - pone + (warp ? wsum64(warp - 1) : 0ull);
  const unsigned long long part_tot = wsum64(31);
  const int total_full = wsum[63];
  int cls_base[4], total_blocks = total_full;
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    cls_base[k] = total_blocks;
    total_blocks += static_cast<int>((part_tot >> (16 * k)) & 0xffffull);
  }
  if (tid < E1) {
    off[tid] = tid < E_local ? rows_excl : P + shared_lo;  // the shared expert's rows follow the routed region, row P + t for token t
    bstart[tid] = full_excl;
    L.counts[tid] = c;
    L.offsets[tid] = off[tid];
    if (tid == E_local) L.offsets[E1] = P + shared_lo + c;
  }
  if (tid == 0) L.nblocks[0] = total_blocks <= max_blocks ? total_blocks : 0;
  __syncthreads();
  for (int p = tid; p < P; p += LISTS_THREADS) {
    const int e = sid[p];
    int row = -1;
    if (e >= 0) {
      row = off[e] + cntw[(p / seg) * E1 + e] + srank[p];
      L.slot_of_row[row] = p;
      L.wt_of_row[row] = wts[p];
    }
    L.row_of_pair[p] = row;
  }
  if (shared_n > 0)
    for (int t = shared_lo + tid; t < shared_lo + shared_n; t += LISTS_THREADS) {
      const bool ok = (pos == nullptr) || (pos[t] != 0);
      L.slot_of_row[P + t] = ok ? P + t : -1;
      L.wt_of_row[P + t] = 1.f;
    }
  if (total_blocks <= max_blocks && tid < E1) {
    int b = bstart[tid];
    for (int j = 0; j < nfull; ++j, ++b) {
      L.blk_expert[b] = tid;
      L.blk_row0[b] = off[tid] + j * block_rows;
      L.blk_rows[b] = min(block_rows, c - j * block_rows);
    }
    if (tail > 0) {
      b = 0;
#pragma unroll
      for (int k = 0; k < 4; ++k)
        if (k == pcls) b = cls_base[k] + static_cast<int>((part_excl >> (16 * k)) & 0xffffull);
      L.blk_expert[b] = tid;
      L.blk_row0[b] = off[tid] + nfull * block_rows;
      L.blk_rows[b] = tail;
    }
  }
}

static size_t lists_smem_bytes(int T, int K, int E_local) {
  const size_t E1 = E_local + 1, P = static_cast<size_t>(T) * K;
  return (E1 + 2 * (E1 + 1) + 128) * 4 + LISTS_WARPS * E1 * 2 + P * 4 + 16;
}

}  // namespace b200

using namespace b200;

// scratch: slice partials [H/128][T][E] fp32
extern "C" size_t b200_router_scratch_bytes(int T, int H, int E) {
  if (T <= 0 || H <= 0 || E <= 0 || H % RT_SLICE || E % RT_EXP) return 0;
  return static_cast<size_t>(H / RT_SLICE) * T * E * sizeof(float);
}

extern "C" int b200_router(const void* x, const float* wr, const float* bias, int T, int H, int E, int K, int flags,
                           float* logits, int32_t* ids, float* wts, void* scratch, size_t scratch_bytes,
                           void* stream) {
  if (!x || !wr || !ids || !wts || !scratch) return fail(B200_E_ARG, "b200_router: null pointer");
  if (T < 0 || H <= 0 || H % RT_SLICE || E <= 0 || E % RT_EXP || E > 1024 || K <= 0 || K > 32 || K > E)
    return fail(B200_E_ARG, "b200_router: need H %% 128 == 0, E %% 64 == 0, E <= 1024, 1 <= K <= 32 (T=%d H=%d E=%d K=%d)",
                T, H, E, K);
  if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(wr) | reinterpret_cast<uintptr_t>(scratch)) & 15)
    return fail(B200_E_ALIGN, "b200_router: x, wr and scratch must be 16-byte aligned");
  if (T == 0) return 0;
  if (scratch_bytes < b200_router_scratch_bytes(T, H, E))
    return fail(B200_E_WS, "b200_router: scratch %zu < %zu bytes", scratch_bytes, b200_router_scratch_bytes(T, H, E));
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  static DeviceOnce once;
  once.run([] {
    cudaFuncSetAttribute(router_partials_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, RtCfg<64>::SMEM);
    cudaFuncSetAttribute(router_partials_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, RtCfg<128>::SMEM);
  });
  float* part = static_cast<float*>(scratch);
  const int nslices = H / RT_SLICE;
  if (T > 64) {
    const int nunits = ((T + 127) / 128) * (E / RT_EXP) * nslices;
    launch_k(router_partials_kernel<128>, dim3(nunits < sm_count() ? nunits : sm_count()), dim3(RT_THREADS), RtCfg<128>::SMEM,
             st, static_cast<const bf16*>(x), wr, T, H, E, part);
  } else {
    const int nunits = (E / RT_EXP) * nslices;
    launch_k(router_partials_kernel<64>, dim3(nunits < sm_count() ? nunits : sm_count()), dim3(RT_THREADS), RtCfg<64>::SMEM,
             st, static_cast<const bf16*>(x), wr, T, H, E, part);
  }
  const int rb = flags & 1;
  const int pl = (E + 127) / 128;
  if (pl <= 1)
    launch_k(router_topk_kernel<1>, dim3(T), dim3(128), 0, st, part, nslices, bias, T, E, K, rb, logits, ids, wts);
  else if (pl <= 2)
    launch_k(router_topk_kernel<2>, dim3(T), dim3(128), 0, st, part, nslices, bias, T, E, K, rb, logits, ids, wts);
  else if (pl <= 4)
    launch_k(router_topk_kernel<4>, dim3(T), dim3(128), 0, st, part, nslices, bias, T, E, K, rb, logits, ids, wts);
  else
    launch_k(router_topk_kernel<8>, dim3(T), dim3(128), 0, st, part, nslices, bias, T, E, K, rb, logits, ids, wts);
  return launch_status("b200_router");
}

// ---------------------------------------------------------------------------------------------------
// Router variant for callers that cannot allocate device memory.
//
// Some hosts of this library are handed nothing but their input and output buffers: a plugin slot
// that a serving engine calls once per decode step has no allocator of its own (the engine planned
// every byte of device memory at start-up and owns the pool), and a cudaMalloc from inside the step
// would stall the whole device or break the engine's memory budget.  For them the slice partials of
// the gate live in the array below instead of a caller-provided scratch buffer.  The array is part
// of the loaded library image: every GPU that loads the library holds these 2 MiB until the process
// exits.  It is shared by all calls and keeps the previous call's partials; nothing in it has to
// start at zero because the gate kernel overwrites every partial the top-k kernel reads.  Two calls
// that overlap on the GPU (different streams, or different host threads) would race on it.
constexpr size_t ROUTER_STATIC_SCRATCH_BYTES = size_t(2) << 20;  // 64 tokens x 512 experts x 16 slices x 4 B
static __device__ __align__(256) unsigned char g_router_static_scratch[ROUTER_STATIC_SCRATCH_BYTES];

extern "C" size_t b200_router_static_max_scratch_bytes(void) { return ROUTER_STATIC_SCRATCH_BYTES; }

extern "C" int b200_router_static(const void* x, const float* wr, const float* bias, int T, int H, int E, int K,
                                  int flags, float* logits, int32_t* ids, float* wts, void* stream) {
  if (T < 0 || H <= 0 || E <= 0 || H % RT_SLICE)
    return fail(B200_E_ARG, "b200_router_static: bad shape (T=%d H=%d E=%d)", T, H, E);
  if (E % RT_EXP) return fail(B200_E_ARG, "b200_router_static: E must be a multiple of 64 (E=%d)", E);
  const size_t need = T == 0 ? 0 : b200_router_scratch_bytes(T, H, E);
  if (need > ROUTER_STATIC_SCRATCH_BYTES)
    return fail(B200_E_WS,
                "b200_router_static: T=%d H=%d E=%d needs %zu bytes of scratch, the built-in scratch holds %zu; "
                "use b200_router with a caller-provided scratch buffer",
                T, H, E, need, ROUTER_STATIC_SCRATCH_BYTES);
  // In host code the array's name is only a handle; the device address is looked up once per device,
  // with that device current, and cached.
  static void* dev_ptr[64] = {nullptr};
  static std::mutex mu;
  int dev = -1;
  cudaError_t err = cudaGetDevice(&dev);
  if (err != cudaSuccess || dev < 0 || dev >= 64)
    return fail(err != cudaSuccess ? static_cast<int>(err) : B200_E_ARG, "b200_router_static: cudaGetDevice failed: %s",
                cudaGetErrorString(err));
  void* scratch = nullptr;
  {
    std::lock_guard<std::mutex> lock(mu);
    if (dev_ptr[dev] == nullptr) {
      void* ptr = nullptr;
      err = cudaGetSymbolAddress(&ptr, g_router_static_scratch);
      if (err != cudaSuccess || ptr == nullptr)
        return fail(err != cudaSuccess ? static_cast<int>(err) : B200_E_DRIVER,
                    "b200_router_static: cudaGetSymbolAddress failed: %s", cudaGetErrorString(err));
      dev_ptr[dev] = ptr;
    }
    scratch = dev_ptr[dev];
  }
  return b200_router(x, wr, bias, T, H, E, K, flags, logits, ids, wts, scratch, ROUTER_STATIC_SCRATCH_BYTES, stream);
}

extern "C" int b200_moe_max_blocks(int T, int K, int E_local, int block_rows) {
  if (T < 0 || K <= 0 || E_local < 0 || block_rows <= 0) return B200_E_ARG;
  // every local expert may end with one partial block; the shared expert adds ceil(T / block_rows)
  return E_local + (T * K) / block_rows + (T + block_rows - 1) / block_rows + 1;
}

extern "C" int b200_moe_build_lists(const int32_t* ids, const float* wts, const int64_t* pos, int T, int K, int e_lo,
                                    int E_local, int block_rows, int with_shared, const b200_moe_lists* lists,
                                    void* stream) {
  return b200_moe_build_lists_range(ids, wts, pos, T, K, e_lo, E_local, block_rows, 0, with_shared ? T : 0, lists, stream);
}

extern "C" int b200_moe_build_lists_range(const int32_t* ids, const float* wts, const int64_t* pos, int T, int K, int e_lo,
                                          int E_local, int block_rows, int shared_lo, int shared_n,
                                          const b200_moe_lists* lists, void* stream) {
  if (!ids || !wts || !lists || !lists->counts || !lists->offsets || !lists->row_of_pair || !lists->slot_of_row ||
      !lists->wt_of_row || !lists->blk_expert || !lists->blk_row0 || !lists->blk_rows || !lists->nblocks)
    return fail(B200_E_ARG, "b200_moe_build_lists: null pointer");
  if (T <= 0 || K <= 0 || E_local <= 0 || E_local > LISTS_MAX_E || e_lo < 0 || block_rows < 16 || block_rows > 128 ||
      block_rows % 16 || shared_lo < 0 || shared_n < 0 || shared_lo + shared_n > T)
    return fail(B200_E_ARG, "b200_moe_build_lists: bad shape (T=%d K=%d E_local=%d block_rows=%d)", T, K, E_local,
                block_rows);
  MoeLists L{lists->counts,     lists->offsets,  lists->row_of_pair, lists->slot_of_row, lists->wt_of_row,
             lists->blk_expert, lists->blk_row0, lists->blk_rows,    lists->nblocks};
  const size_t smem = lists_smem_bytes(T, K, E_local);
  if (smem > 200 * 1024 || T * (K + 1) > 65535 * 4)
    return fail(B200_E_ARG, "b200_moe_build_lists: T*K = %d is above the single-CTA limit", T * K);
  static DeviceOnce once;
  once.run([] { cudaFuncSetAttribute(moe_lists_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024); });
  launch_k(moe_lists_kernel, dim3(1), dim3(LISTS_THREADS), smem, static_cast<cudaStream_t>(stream), ids, wts, pos, T, K,
           e_lo, E_local, block_rows, shared_lo, shared_n, static_cast<int>(b200_moe_max_blocks(T, K, E_local, block_rows)), L);
  return launch_status("b200_moe_build_lists");
}
