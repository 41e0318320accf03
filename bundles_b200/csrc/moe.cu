// MoE block: activation quantise + permute, grouped expert GEMMs on tcgen05 tensor cores with
// TMEM accumulators and TMA-fed shared-memory rings, SwiGLU / unpermute epilogues, combine.
//
// Replaces the reference's decode MoE (i8x_decode.py:528-576 moe_row_batch; qk_moe_up16.cu:139
// up_kernel, qk_moe_dn16.cu:136 down_kernel, qk_route.cu:686 combine_norm_kernel) at the target
// formats (int8 W8A8: qk_moe_prefill_i8.cu:3646-3655,4061-4071; fp8 128x128 block scales).
//
// GEMM orientation (the reference's "weights as the MMA M side", qk_moe_up16.cu:9): one UMMA is
// M = 128 weight rows x N = 16..128 tokens of one expert x K = 32 bytes.  Weights arrive by 2-D TMA
// straight from the expert tensors ([rows, K] bytes, 128-byte swizzle); tokens were permuted into
// expert-sorted rows by the quantise kernel, so the token operand is a plain 2-D TMA box as well.
// A CTA is persistent and walks (block, 128-row weight tile) pairs: warp 0 issues TMA, warp 1 issues
// MMAs and owns the TMEM allocation, warps 2-9 drain TMEM (two per 32-lane quadrant).
// At decode sizes this path is bound by the HBM stream of expert weights, not by the tensor pipe.
#include "common.cuh"
#include "host.h"

namespace b200 {

B200_DEFINE_WAIT_BUDGET_SETTER(set_wait_budget_moe)

// ---------------------------------------------------------------------------------------------------
// activation quantise + permute (int8): one CTA per token
// ---------------------------------------------------------------------------------------------------
__device__ __forceinline__ float block_max(float v, float* red) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(FULL_MASK, v, o));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float r = lane < nw ? red[lane] : 0.f;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) r = fmaxf(r, __shfl_xor_sync(FULL_MASK, r, o));
  __syncthreads();
  return r;
}

// round half away from zero, clamp to +-127 (qwen36_lmhead8/w8a8.py:15-22)
__device__ __forceinline__ int q8(float x, float safe) {
  const float v = __fdiv_rn(x, safe);
  float r = v >= 0.f ? floorf(v + 0.5f) : -floorf(0.5f - v);
  r = fminf(fmaxf(r, -127.f), 127.f);
  return static_cast<int>(r);
}

// x bf16 [T, H] -> int8 rows written at every sorted row of the token (its K routed rows and its
// shared-expert row), scale per row.  256 threads, 8 elements per thread per pass.
__global__ void __launch_bounds__(256) quant_permute_i8_kernel(const bf16* __restrict__ x, int T, int H, int K,
                                                               const int32_t* __restrict__ row_of_pair,
                                                               int shared_lo, int shared_n, int8_t* __restrict__ xq,
                                                               float* __restrict__ xs) {
  __shared__ float red[8];
  __shared__ int rows[40];
  const int t = blockIdx.x, tid = threadIdx.x;
  pdl_wait();
  pdl_launch();
  if (tid < K) rows[tid] = row_of_pair[t * K + tid];
  if (tid == K) rows[K] = (t >= shared_lo && t < shared_lo + shared_n) ? T * K + t : -1;
  const bf16* xr = x + static_cast<size_t>(t) * H;
  float amax = 0.f;
  for (int c = tid * 8; c < H; c += 256 * 8) {
    const uint4 v = *reinterpret_cast<const uint4*>(xr + c);
    amax = fmaxf(amax, fmaxf(fmaxf(fabsf(bf_lo(v.x)), fabsf(bf_hi(v.x))), fmaxf(fabsf(bf_lo(v.y)), fabsf(bf_hi(v.y)))));
    amax = fmaxf(amax, fmaxf(fmaxf(fabsf(bf_lo(v.z)), fabsf(bf_hi(v.z))), fmaxf(fabsf(bf_lo(v.w)), fabsf(bf_hi(v.w)))));
  }
  amax = block_max(amax, red);
  const float scale = __fdiv_rn(amax, 127.f);
  const float safe = amax > 0.f ? scale : 1.f;
  for (int c = tid * 8; c < H; c += 256 * 8) {
    const uint4 v = *reinterpret_cast<const uint4*>(xr + c);
    const float f[8] = {bf_lo(v.x), bf_hi(v.x), bf_lo(v.y), bf_hi(v.y), bf_lo(v.z), bf_hi(v.z), bf_lo(v.w), bf_hi(v.w)};
    uint32_t lo = 0, hi = 0;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      lo |= (static_cast<uint32_t>(q8(f[i], safe)) & 0xffu) << (8 * i);
      hi |= (static_cast<uint32_t>(q8(f[4 + i], safe)) & 0xffu) << (8 * i);
    }
    for (int j = 0; j <= K; ++j) {
      const int row = rows[j];
      if (row >= 0) *reinterpret_cast<uint2*>(xq + static_cast<size_t>(row) * H + c) = make_uint2(lo, hi);
    }
  }
  if (tid <= K && rows[tid] >= 0) xs[rows[tid]] = scale;
}

// h bf16 [rows, I] -> int8 + per-row scale (the re-quantisation before the down GEMM,
// qk_moe_prefill_i8.cu:4061-4066).  One warp per sorted row; rows without a slot are skipped.
__global__ void __launch_bounds__(256) quant_rows_i8_kernel(const bf16* __restrict__ h, int rows, int I,
                                                            const int32_t* __restrict__ slot_of_row,
                                                            int8_t* __restrict__ hq, float* __restrict__ hs) {
  const int row = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  pdl_wait();
  pdl_launch();
  if (row >= rows) return;
  const bf16* hr = h + static_cast<size_t>(row) * I;
  // I <= 1024: the row is read once, all loads in flight together with the slot lookup (every sorted row below
  // `rows` is readable memory; a row without a slot is simply not written)
  constexpr int MAXV = 4;
  const bool fits = I <= MAXV * 256;
  uint4 v[MAXV];
  if (fits) {
#pragma unroll
    for (int i = 0; i < MAXV; ++i)
      v[i] = lane * 8 + i * 256 < I ? *reinterpret_cast<const uint4*>(hr + lane * 8 + i * 256) : make_uint4(0u, 0u, 0u, 0u);
  }
  if (slot_of_row[row] < 0) return;
  float amax = 0.f;
  auto absmax = [&](const uint4& q) {
    amax = fmaxf(amax, fmaxf(fmaxf(fabsf(bf_lo(q.x)), fabsf(bf_hi(q.x))), fmaxf(fabsf(bf_lo(q.y)), fabsf(bf_hi(q.y)))));
    amax = fmaxf(amax, fmaxf(fmaxf(fabsf(bf_lo(q.z)), fabsf(bf_hi(q.z))), fmaxf(fabsf(bf_lo(q.w)), fabsf(bf_hi(q.w)))));
  };
  if (fits) {
#pragma unroll
    for (int i = 0; i < MAXV; ++i) absmax(v[i]);
  } else {
    for (int c = lane * 8; c < I; c += 256) absmax(*reinterpret_cast<const uint4*>(hr + c));
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(FULL_MASK, amax, o));
  const float scale = __fdiv_rn(amax, 127.f);
  const float safe = amax > 0.f ? scale : 1.f;
  auto emit = [&](const uint4& q, int c) {
    const float f[8] = {bf_lo(q.x), bf_hi(q.x), bf_lo(q.y), bf_hi(q.y), bf_lo(q.z), bf_hi(q.z), bf_lo(q.w), bf_hi(q.w)};
    uint32_t lo = 0, hi = 0;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      lo |= (static_cast<uint32_t>(q8(f[i], safe)) & 0xffu) << (8 * i);
      hi |= (static_cast<uint32_t>(q8(f[4 + i], safe)) & 0xffu) << (8 * i);
    }
    *reinterpret_cast<uint2*>(hq + static_cast<size_t>(row) * I + c) = make_uint2(lo, hi);
  };
  if (fits) {
#pragma unroll
    for (int i = 0; i < MAXV; ++i)
      if (lane * 8 + i * 256 < I) emit(v[i], lane * 8 + i * 256);
  } else {
    for (int c = lane * 8; c < I; c += 256) emit(*reinterpret_cast<const uint4*>(hr + c), c);
  }
  if (lane == 0) hs[row] = scale;
}

// ---------------------------------------------------------------------------------------------------
// grouped int8 GEMM on tcgen05 (kind::i8), swap-AB
// ---------------------------------------------------------------------------------------------------
struct GemmArgs {
  MoeLists L;
  int E_local;      // local routed experts; block expert == E_local means the shared expert
  int mtiles;       // 128-row weight tiles per expert (up: I/128, down: H/128)
  int ksteps;       // K / 128
  int w_rows;       // weight rows per expert (up: 2I, down: H)
  int I, H;
  int total_rows;   // T * (K + 1)
  const float* s_w;     // routed weight scales [E_local, w_rows]
  const float* s_w_sh;  // shared-expert weight scales [w_rows]
  const float* a_scale; // activation scale per sorted row
  bf16* h_out;          // up: SwiGLU output, sorted rows [total_rows, I]
  bf16* cache;          // down: [total_rows, H] by slot
  int32_t* dbg_acc;     // up: raw accumulators by slot [total_rows, 2I] or null
  bf16* dbg_h;          // up: h by slot or null
  int32_t* status;
  // expert-parallel down epilogue: routed slot s of the gathered batch belongs to rank s / ep_rows, whose
  // cache (this GPU's own, or a peer's mapped over NVLink) receives the row at local slot s % ep_rows
  int ep_world;         // 0 / 1: single GPU, rows go to `cache`
  int ep_rows;          // routed slots per rank = tokens per rank x top-k
  int ep_rank, ep_tokens;  // this rank and tokens per rank: shared-expert rows are kept only for own tokens
  bf16* ep_cache[8];
  int test_starve;  // self-test: the producer leaves out the token rows, so no stage ever completes and every wait runs out
};

constexpr int TILE_BYTES = 128 * 128;   // one 128-row x 128-byte operand tile
constexpr int GEMM_THREADS = 320;   // TMA warp, MMA warp, 8 epilogue warps (two per TMEM lane quadrant)
constexpr int TMEM_COLS = 512;
constexpr int I8_CACHED = 64;       // tiles per CTA whose list entries are cached in shared memory

template <bool UP>
struct GemmCfg {
  static constexpr int NA = 2;   // weight tiles per stage: gate + up rows of one channel block / two consecutive 128-row tiles of W2
  static constexpr int STAGE = NA * TILE_BYTES + TILE_BYTES;  // + token tile (<= 128 rows)
  static constexpr int STAGES = 4;
  static constexpr int SMEM = STAGES * STAGE + 1024 /*align*/ + 256 /*barriers*/ + 8 * 128 * 20 /*row metadata, one copy per epilogue warp*/ +
                              I8_CACHED * 12 /*block-list entries of this CTA's tiles*/;
};

template <bool UP>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
moe_gemm_i8_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmWsh,
                   const __grid_constant__ CUtensorMap tmX, const __grid_constant__ CUtensorMap tmX64,
                   const __grid_constant__ CUtensorMap tmX128, const GemmArgs p) {
  using C = GemmCfg<UP>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + C::STAGES * C::STAGE);
  uint64_t* empty = full + C::STAGES;
  uint64_t* tfull = empty + C::STAGES;
  uint64_t* tempty = tfull + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  // per-tile row metadata for the epilogue: each epilogue warp keeps its own copy, so no barrier
  // between warps is needed (a warp-private buffer is refilled only after that warp is done with it)
  float* m_scale_all = reinterpret_cast<float*>(smem + C::STAGES * C::STAGE + 256);  // [8][128] activation scale
  float* m_wt_all = m_scale_all + 1024;                                               // [8][128] routing weight
  int* m_slot_all = reinterpret_cast<int*>(m_wt_all + 1024);                          // [8][128] slot or -1
  bf16** m_dst_all = reinterpret_cast<bf16**>(m_slot_all + 1024);                     // [8][128] destination row (down)
  int* binfo = reinterpret_cast<int*>(m_dst_all + 1024);                              // [I8_CACHED][3] expert, row0, rows

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int s = 0; s < C::STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&tfull[b], 1);
      mbar_init(&tempty[b], 8);
    }
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmW);
    tma_prefetch_desc(&tmWsh);
    tma_prefetch_desc(&tmX);
    tma_prefetch_desc(&tmX64);
    tma_prefetch_desc(&tmX128);
  }
  // Tiles are (block, 128-row weight tile) pairs; CTA b takes tiles b, b + grid, ... (hot and cold blocks mix
  // evenly).  With every pipeline stage in flight a dependent global load costs microseconds (it queues
  // behind the weight stream), so nothing on the per-tile path may wait for one: the list entries of this
  // CTA's tiles are read into shared memory before the stream starts, and the epilogue's row metadata
  // and weight scales are loaded one tile ahead.
  const int nblocks = p.L.nblocks[0];
  const int ntiles = nblocks * p.mtiles;
  if (threadIdx.x < I8_CACHED) {
    const int tile = blockIdx.x + threadIdx.x * gridDim.x;
    if (tile < ntiles) {
      const int blk = tile / p.mtiles;
      binfo[threadIdx.x * 3 + 0] = p.L.blk_expert[blk];
      binfo[threadIdx.x * 3 + 1] = p.L.blk_row0[blk];
      binfo[threadIdx.x * 3 + 2] = p.L.blk_rows[blk];
    }
  }
  if (warp == 1) tmem_alloc(tmem_slot, TMEM_COLS);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  // every role decodes a tile the same way; a malformed list entry is skipped by all of them
  auto decode = [&](int tile, int& e, int& row0, int& n, int& mt) -> bool {
    const int blk = tile / p.mtiles;
    mt = tile - blk * p.mtiles;
    const int ci = (tile - static_cast<int>(blockIdx.x)) / static_cast<int>(gridDim.x);
    if (ci < I8_CACHED) {
      e = binfo[ci * 3 + 0];
      row0 = binfo[ci * 3 + 1];
      n = binfo[ci * 3 + 2];
    } else {
      e = p.L.blk_expert[blk];
      row0 = p.L.blk_row0[blk];
      n = p.L.blk_rows[blk];
    }
    return e >= 0 && e <= p.E_local && n >= 1 && n <= 128 && row0 >= 0 && row0 + n <= p.total_rows;
  };

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      int issued = 0;
      bool ok = true;
      // every TMA instruction costs the issuing thread ~80 ns, so the token rows come in as few boxes as
      // possible: 16-row boxes up to 32 rows, one 64-row box (+ up to two 16-row boxes), or one 128-row
      // box.  Rows past the block belong to the next expert or are zero-filled past the end of the
      // tensor; the MMA's N ignores them.
      auto big_of = [](int nb16) { return nb16 > 6 ? 8 : (nb16 > 2 ? 4 : 0); };  // 16-row units in the large box
      auto tok_units = [&](int nb16) { const int big = big_of(nb16); return nb16 > big ? nb16 : big; };
      // The weights do not depend on the kernels before this one: the first stages' weight tiles are requested
      // before the dependency wait, the token rows of the same stages after it.
      int pre = 0;
      for (int tile = blockIdx.x; pre < C::STAGES && tile < ntiles; tile += gridDim.x) {
        int e, row0, n, mt;
        if (!decode(tile, e, row0, n, mt)) continue;
        const CUtensorMap* mapW = (e == p.E_local) ? &tmWsh : &tmW;
        const int wrow = (e == p.E_local ? 0 : e * p.w_rows) + mt * (UP ? 128 : 256);
        for (int ks = 0; ks < p.ksteps && pre < C::STAGES; ++ks, ++pre) {
          uint8_t* sA = smem + pre * C::STAGE;
          mbar_expect_tx(&full[pre], C::NA * TILE_BYTES + tok_units((n + 15) >> 4) * 2048);
          tma_load_2d(sA, mapW, ks * 128, wrow, &full[pre]);
          tma_load_2d(sA + TILE_BYTES, mapW, ks * 128, wrow + (UP ? p.I : 128), &full[pre]);
        }
      }
      pdl_wait();
      pdl_launch();
      for (int tile = blockIdx.x; ok && tile < ntiles; tile += gridDim.x) {
        int e, row0, n, mt;
        if (!decode(tile, e, row0, n, mt)) continue;
        const int nb16 = (n + 15) >> 4;
        const CUtensorMap* mapW = (e == p.E_local) ? &tmWsh : &tmW;
        const int wrow = (e == p.E_local ? 0 : e * p.w_rows) + mt * (UP ? 128 : 256);
        for (int ks = 0; ks < p.ksteps; ++ks) {
          uint8_t* sA = smem + stage * C::STAGE;
          uint8_t* sB = sA + C::NA * TILE_BYTES;
          const int big = big_of(nb16);
          if (issued >= pre) {
            if (!mbar_wait(&empty[stage], phase ^ 1u, abort_flag, p.status, ST_WAIT_EMPTY)) {
              ok = false;
              break;
            }
            mbar_expect_tx(&full[stage], C::NA * TILE_BYTES + tok_units(nb16) * 2048);
            tma_load_2d(sA, mapW, ks * 128, wrow, &full[stage]);
            tma_load_2d(sA + TILE_BYTES, mapW, ks * 128, wrow + (UP ? p.I : 128), &full[stage]);
          }
          if (!p.test_starve) {
            if (big == 8) tma_load_2d(sB, &tmX128, ks * 128, row0, &full[stage]);
            if (big == 4) tma_load_2d(sB, &tmX64, ks * 128, row0, &full[stage]);
            for (int b = big; b < nb16; ++b) tma_load_2d(sB + b * 2048, &tmX, ks * 128, row0 + 16 * b, &full[stage]);
          }
          ++issued;
          if (++stage == C::STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
      if (!ok) {
        // abandoned: give the copies already in flight a bounded time to land before the CTA exits
        const unsigned long long t0 = globaltimer();
        const int back = issued < C::STAGES ? issued : C::STAGES;
        for (int i = 1; i <= back; ++i) {
          int s = stage - i;
          uint32_t ph = phase;
          if (s < 0) {
            s += C::STAGES;
            ph ^= 1u;
          }
          while (!mbar_try(&full[s], ph) && globaltimer() - t0 < 20000000ull) {
          }
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    pdl_wait();
    pdl_launch();
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      int it = 0;
      bool ok = true;
      for (int tile = blockIdx.x; ok && tile < ntiles; tile += gridDim.x) {
        int e, row0, n, mt;
        if (!decode(tile, e, row0, n, mt)) continue;
        const int buf = it & 1;
        const uint32_t bphase = (it >> 1) & 1;
        ++it;
        if (!mbar_wait(&tempty[buf], bphase ^ 1u, abort_flag, p.status, ST_WAIT_TMEM_EMPTY)) break;
        tc_fence_after();
        const uint32_t N = static_cast<uint32_t>((n + 15) & ~15);
        const uint32_t idesc = umma_idesc(UMMA_C_S32, UMMA_AB_INT8, N);
        const uint32_t d0 = tmem_base + buf * 256;
        for (int ks = 0; ks < p.ksteps; ++ks) {
          if (!mbar_wait(&full[stage], phase, abort_flag, p.status, ST_WAIT_FULL)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sA = smem_u32(smem + stage * C::STAGE);
          const uint32_t sB = sA + C::NA * TILE_BYTES;
#pragma unroll
          for (int kk = 0; kk < 4; ++kk) {
            const uint64_t db = umma_desc_sw128(sB + kk * 32);
            const uint32_t acc = (ks | kk) != 0;
            tc_mma_i8(d0, umma_desc_sw128(sA + kk * 32), db, idesc, acc);
            tc_mma_i8(d0 + 128, umma_desc_sw128(sA + TILE_BYTES + kk * 32), db, idesc, acc);
          }
          tc_commit(&empty[stage]);
          if (++stage == C::STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (ok) tc_commit(&tfull[buf]);
      }
    }
  } else {
    // ---------------- epilogue: warps 2..9; TMEM lane quadrant = warp % 4, and the two warps of a quadrant
    // (they share a scheduler, so one covers the other's TMEM and memory latencies) take alternate
    // 16-column chunks of the tile ----------------
    const int q = warp & 3;
    const int half = (warp - 2) >> 2;
    float* ms = m_scale_all + (warp - 2) * 128;
    float* m_wt = m_wt_all + (warp - 2) * 128;
    int* m_slot = m_slot_all + (warp - 2) * 128;
    bf16** m_dst = m_dst_all + (warp - 2) * 128;
    const float* __restrict__ a_scale = p.a_scale;
    const float* __restrict__ wt_of_row = p.L.wt_of_row;
    const int32_t* __restrict__ slot_of_row = p.L.slot_of_row;
    int it = 0;
    // everything the epilogue of a tile reads from global memory, loaded one tile ahead into registers:
    // activation scale, slot and routing weight of columns lane, lane + 32, ..., and the weight scale(s)
    // of this lane's row.  No loaded value is consumed where it is fetched.
    struct Pre {
      float sc[4], wt[4], w0, w1;
      int sl[4];
    };
    const int step = static_cast<int>(gridDim.x);
    auto fetch = [&](int tile, Pre& m) {
      m.w0 = m.w1 = 0.f;
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        m.sc[u] = m.wt[u] = 0.f;
        m.sl[u] = -1;
      }
      int e, row0, n, mt;
      if (tile >= ntiles || !decode(tile, e, row0, n, mt)) return;
      const float* sw = (e == p.E_local) ? p.s_w_sh : p.s_w + static_cast<size_t>(e) * p.w_rows;
      const int r = mt * (UP ? 128 : 256) + q * 32 + lane;
      m.w0 = sw[r];
      m.w1 = sw[(UP ? p.I : 128) + r];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int c = lane + 32 * u;
        if (c < n) {
          m.sc[u] = a_scale[row0 + c];
          m.sl[u] = slot_of_row[row0 + c];
          if (!UP) m.wt[u] = wt_of_row[row0 + c];
        }
      }
    };
    Pre pre;
    pdl_wait();
    pdl_launch();
    fetch(blockIdx.x, pre);
    for (int tile = blockIdx.x; tile < ntiles; tile += step) {
      int e, row0, n, mt;
      const float ws0 = pre.w0, ws1 = pre.w1;
      const bool good = decode(tile, e, row0, n, mt);
      if (good) {
        // stage this tile's row metadata (entries past n only pad the last 16-column chunk)
        __syncwarp();
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int c = lane + 32 * u;
          int slot = pre.sl[u];
          if (slot >= p.total_rows) slot = -1;
          ms[c] = pre.sc[u];
          m_wt[c] = pre.wt[u];
          m_slot[c] = slot;
          if (!UP) {
            bf16* dst = nullptr;
            if (slot >= 0) {
              if (p.ep_world >= 1) {
                const int routed = p.ep_rows * p.ep_world;
                if (slot < routed) {
                  const int home = slot / p.ep_rows;
                  dst = p.ep_cache[home] + static_cast<size_t>(slot - home * p.ep_rows) * p.H;
                } else {  // shared-expert row of token t: kept at row ep_rows + local t of this rank's own cache
                  const int t = slot - routed, home = t / p.ep_tokens;
                  if (home == p.ep_rank)
                    dst = p.ep_cache[home] + static_cast<size_t>(p.ep_rows + t - home * p.ep_tokens) * p.H;
                }
              } else {
                dst = p.cache + static_cast<size_t>(slot) * p.H;
              }
            }
            m_dst[c] = dst;
          }
        }
        __syncwarp();
      }
      fetch(tile + step, pre);  // in flight during this tile's epilogue
      if (!good) {
        if (lane == 0 && p.status) atomicCAS(p.status, 0, ST_BAD_LIST);
        continue;
      }
      const int buf = it & 1;
      const uint32_t bphase = (it >> 1) & 1;
      ++it;
      if (!mbar_wait(&tfull[buf], bphase, abort_flag, p.status, ST_WAIT_TMEM_FULL)) break;
      tc_fence_after();
      const uint32_t taddr = tmem_base + buf * 256 + (static_cast<uint32_t>(q * 32) << 16);
      const int r = mt * (UP ? 128 : 256) + q * 32 + lane;  // weight row inside the expert (up: channel of I; down: column of H, and r + 128)
      if (UP) {
        const float wsg = ws0, wsu = ws1;
        bf16* __restrict__ hout = p.h_out + static_cast<size_t>(row0) * p.I + r;
        for (int c0 = half * 16; c0 < n; c0 += 32) {
          uint32_t rg[16], ru[16];
          tmem_ld16(taddr + c0, rg);
          tmem_ld16(taddr + 128 + c0, ru);
          tmem_ld_wait();
          bf16 hv[16];
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            const float xs = ms[c0 + i];
            const float g = rbf(__fmul_rn(__fmul_rn(static_cast<float>(static_cast<int>(rg[i])), xs), wsg));
            const float u = rbf(__fmul_rn(__fmul_rn(static_cast<float>(static_cast<int>(ru[i])), xs), wsu));
            hv[i] = f2bf(__fmul_rn(__fdividef(g, 1.f + __expf(-g)), u));
          }
#pragma unroll
          for (int i = 0; i < 16; ++i)
            if (c0 + i < n) st_global_na(hout + static_cast<size_t>(c0 + i) * p.I, hv[i]);
          if (p.dbg_acc || p.dbg_h) {
#pragma unroll
            for (int i = 0; i < 16; ++i) {
              const int slot = c0 + i < n ? m_slot[c0 + i] : -1;
              if (slot >= 0) {
                if (p.dbg_acc) {
                  p.dbg_acc[static_cast<size_t>(slot) * 2 * p.I + r] = static_cast<int>(rg[i]);
                  p.dbg_acc[static_cast<size_t>(slot) * 2 * p.I + p.I + r] = static_cast<int>(ru[i]);
                }
                if (p.dbg_h) p.dbg_h[static_cast<size_t>(slot) * p.I + r] = hv[i];
              }
            }
          }
        }
      } else {
        for (int c0 = half * 16; c0 < n; c0 += 32) {
          uint32_t ra[16], rb[16];  // output columns r and r + 128 of the same token rows
          tmem_ld16(taddr + c0, ra);
          tmem_ld16(taddr + 128 + c0, rb);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            bf16* dst = m_dst[c0 + i];
            const float xs = ms[c0 + i], wt = m_wt[c0 + i];
            const float y0 = __fmul_rn(__fmul_rn(static_cast<float>(static_cast<int>(ra[i])), xs), ws0);
            const float y1 = __fmul_rn(__fmul_rn(static_cast<float>(static_cast<int>(rb[i])), xs), ws1);
            if (dst != nullptr) {
              st_global_na(dst + r, f2bf(__fmul_rn(y0, wt)));
              st_global_na(dst + r + 128, f2bf(__fmul_rn(y1, wt)));
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty[buf]);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// ---------------------------------------------------------------------------------------------------
// combine
// ---------------------------------------------------------------------------------------------------
// One CTA per token, 256 threads, 8 columns per thread per pass.  gate = sigmoid(x . gate_w) in fp32
// (i8x_decode.py:436-438); out = bf16(sum of the K routed rows in slot order + gate * shared row).
__global__ void __launch_bounds__(256) moe_combine_kernel(const bf16* __restrict__ cache, const bf16* __restrict__ x,
                                                          const bf16* __restrict__ gate_w,
                                                          const int64_t* __restrict__ pos, int T, int H, int K,
                                                          bf16* __restrict__ out) {
  __shared__ float red[8];
  const int t = blockIdx.x, tid = threadIdx.x;
  pdl_wait();
  pdl_launch();
  bf16* orow = out + static_cast<size_t>(t) * H;
  if (pos != nullptr && pos[t] == 0) {
    for (int c = tid * 8; c < H; c += 2048) *reinterpret_cast<uint4*>(orow + c) = make_uint4(0, 0, 0, 0);
    return;
  }
  float gate = 0.f;
  if (gate_w != nullptr) {
    float dot = 0.f;
    for (int c = tid * 8; c < H; c += 2048) {
      const uint4 a = *reinterpret_cast<const uint4*>(x + static_cast<size_t>(t) * H + c);
      const uint4 w = *reinterpret_cast<const uint4*>(gate_w + c);
      dot = fmaf(bf_lo(a.x), bf_lo(w.x), dot); dot = fmaf(bf_hi(a.x), bf_hi(w.x), dot);
      dot = fmaf(bf_lo(a.y), bf_lo(w.y), dot); dot = fmaf(bf_hi(a.y), bf_hi(w.y), dot);
      dot = fmaf(bf_lo(a.z), bf_lo(w.z), dot); dot = fmaf(bf_hi(a.z), bf_hi(w.z), dot);
      dot = fmaf(bf_lo(a.w), bf_lo(w.w), dot); dot = fmaf(bf_hi(a.w), bf_hi(w.w), dot);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) dot += __shfl_xor_sync(FULL_MASK, dot, o);
    if ((tid & 31) == 0) red[tid >> 5] = dot;
    __syncthreads();
    float s = 0.f;
    for (int w = 0; w < 8; ++w) s += red[w];
    gate = 1.f / (1.f + __expf(-s));
  }
  for (int c = tid * 8; c < H; c += 2048) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int j = 0; j < K; ++j) {
      const uint4 v = *reinterpret_cast<const uint4*>(cache + (static_cast<size_t>(t) * K + j) * H + c);
      acc[0] += bf_lo(v.x); acc[1] += bf_hi(v.x); acc[2] += bf_lo(v.y); acc[3] += bf_hi(v.y);
      acc[4] += bf_lo(v.z); acc[5] += bf_hi(v.z); acc[6] += bf_lo(v.w); acc[7] += bf_hi(v.w);
    }
    if (gate_w != nullptr) {
      const uint4 v = *reinterpret_cast<const uint4*>(cache + (static_cast<size_t>(T) * K + t) * H + c);
      acc[0] += gate * bf_lo(v.x); acc[1] += gate * bf_hi(v.x); acc[2] += gate * bf_lo(v.y); acc[3] += gate * bf_hi(v.y);
      acc[4] += gate * bf_lo(v.z); acc[5] += gate * bf_hi(v.z); acc[6] += gate * bf_lo(v.w); acc[7] += gate * bf_hi(v.w);
    }
    *reinterpret_cast<uint4*>(orow + c) = make_uint4(pack_bf2(acc[0], acc[1]), pack_bf2(acc[2], acc[3]),
                                                     pack_bf2(acc[4], acc[5]), pack_bf2(acc[6], acc[7]));
  }
}

// The combine with the next layer's input norm folded in (the reference's combine_norm_kernel, qk_route.cu:686-820):
// out as above; r = bf16(out + residual) written back to `residual`; y = bf16(r * rsqrt(mean r^2 + eps) * (1 + w)).
// Same arithmetic, in the same order, as moe_combine_kernel followed by add_rmsnorm_kernel.
__global__ void __launch_bounds__(256) moe_combine_norm_kernel(const bf16* __restrict__ cache, const bf16* __restrict__ x,
                                                               const bf16* __restrict__ gate_w,
                                                               const int64_t* __restrict__ pos, int T, int H, int K,
                                                               bf16* __restrict__ out, bf16* __restrict__ residual,
                                                               const bf16* __restrict__ norm_w, float eps,
                                                               bf16* __restrict__ normed, uint8_t* __restrict__ xq_out,
                                                               float* __restrict__ xs_out) {
  __shared__ float red[8], red2[8];
  const int t = blockIdx.x, tid = threadIdx.x;
  pdl_wait();
  pdl_launch();
  const bool pad = pos != nullptr && pos[t] == 0;
  // H == 2048 and K <= 12 (the decode shapes): a thread owns 8 columns, and everything it reads (its x and gate
  // columns, the K + 1 cache rows, the residual, the norm weight) is requested before anything is used: one round
  // trip to memory instead of three.  The arithmetic and its order are those of the general path below.
  if (H == 2048 && K <= 12) {
    const int c = tid * 8;
    const uint4 zero4 = make_uint4(0u, 0u, 0u, 0u);
    const bool gated = gate_w != nullptr;
    const uint4 xa = (!pad && gated) ? *reinterpret_cast<const uint4*>(x + static_cast<size_t>(t) * H + c) : zero4;
    const uint4 gw4 = (!pad && gated) ? *reinterpret_cast<const uint4*>(gate_w + c) : zero4;
    uint4 rows[13];
#pragma unroll
    for (int j = 0; j < 12; ++j)
      rows[j] = (!pad && j < K) ? *reinterpret_cast<const uint4*>(cache + (static_cast<size_t>(t) * K + j) * H + c) : zero4;
    rows[12] = (!pad && gated) ? *reinterpret_cast<const uint4*>(cache + (static_cast<size_t>(T) * K + t) * H + c) : zero4;
    const uint4 b = *reinterpret_cast<const uint4*>(residual + static_cast<size_t>(t) * H + c);
    const uint4 g = *reinterpret_cast<const uint4*>(norm_w + c);
    float gate = 0.f;
    if (!pad && gated) {
      float dot = 0.f;
      dot = fmaf(bf_lo(xa.x), bf_lo(gw4.x), dot); dot = fmaf(bf_hi(xa.x), bf_hi(gw4.x), dot);
      dot = fmaf(bf_lo(xa.y), bf_lo(gw4.y), dot); dot = fmaf(bf_hi(xa.y), bf_hi(gw4.y), dot);
      dot = fmaf(bf_lo(xa.z), bf_lo(gw4.z), dot); dot = fmaf(bf_hi(xa.z), bf_hi(gw4.z), dot);
      dot = fmaf(bf_lo(xa.w), bf_lo(gw4.w), dot); dot = fmaf(bf_hi(xa.w), bf_hi(gw4.w), dot);
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) dot += __shfl_xor_sync(FULL_MASK, dot, o);
      if ((tid & 31) == 0) red[tid >> 5] = dot;
    }
    __syncthreads();
    if (!pad && gated) {
      float s = 0.f;
      for (int w = 0; w < 8; ++w) s += red[w];
      gate = 1.f / (1.f + __expf(-s));
    }
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    if (!pad) {
#pragma unroll
      for (int j = 0; j < 12; ++j)
        if (j < K) {
          const uint4 v = rows[j];
          acc[0] += bf_lo(v.x); acc[1] += bf_hi(v.x); acc[2] += bf_lo(v.y); acc[3] += bf_hi(v.y);
          acc[4] += bf_lo(v.z); acc[5] += bf_hi(v.z); acc[6] += bf_lo(v.w); acc[7] += bf_hi(v.w);
        }
      if (gated) {
        const uint4 v = rows[12];
        acc[0] += gate * bf_lo(v.x); acc[1] += gate * bf_hi(v.x); acc[2] += gate * bf_lo(v.y); acc[3] += gate * bf_hi(v.y);
        acc[4] += gate * bf_lo(v.z); acc[5] += gate * bf_hi(v.z); acc[6] += gate * bf_lo(v.w); acc[7] += gate * bf_hi(v.w);
      }
    }
    const uint4 o4 = make_uint4(pack_bf2(acc[0], acc[1]), pack_bf2(acc[2], acc[3]), pack_bf2(acc[4], acc[5]),
                                pack_bf2(acc[6], acc[7]));
    if (out != nullptr) *reinterpret_cast<uint4*>(out + static_cast<size_t>(t) * H + c) = o4;
    float r[8] = {rbf(bf_lo(o4.x) + bf_lo(b.x)), rbf(bf_hi(o4.x) + bf_hi(b.x)), rbf(bf_lo(o4.y) + bf_lo(b.y)),
                  rbf(bf_hi(o4.y) + bf_hi(b.y)), rbf(bf_lo(o4.z) + bf_lo(b.z)), rbf(bf_hi(o4.z) + bf_hi(b.z)),
                  rbf(bf_lo(o4.w) + bf_lo(b.w)), rbf(bf_hi(o4.w) + bf_hi(b.w))};
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) ss = fmaf(r[i], r[i], ss);
    *reinterpret_cast<uint4*>(residual + static_cast<size_t>(t) * H + c) =
        make_uint4(pack_bf2(r[0], r[1]), pack_bf2(r[2], r[3]), pack_bf2(r[4], r[5]), pack_bf2(r[6], r[7]));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(FULL_MASK, ss, o);
    if ((tid & 31) == 0) red2[tid >> 5] = ss;
    __syncthreads();
    float tot = 0.f;
    for (int i = 0; i < 8; ++i) tot += red2[i];
    const float rstd = rsqrtf(tot / H + eps);
    const float gwn[8] = {bf_lo(g.x), bf_hi(g.x), bf_lo(g.y), bf_hi(g.y), bf_lo(g.z), bf_hi(g.z), bf_lo(g.w), bf_hi(g.w)};
    float y[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) y[i] = r[i] * rstd * (1.f + gwn[i]);
    const uint4 y4 = make_uint4(pack_bf2(y[0], y[1]), pack_bf2(y[2], y[3]), pack_bf2(y[4], y[5]), pack_bf2(y[6], y[7]));
    *reinterpret_cast<uint4*>(normed + static_cast<size_t>(t) * H + c) = y4;
    if (xq_out != nullptr) {
      // the normed row also leaves in the e4m3 form the next projection reads (the arithmetic of
      // quant_permute_f8_kernel: 16 consecutive threads own one 128-channel group)
      float amax = amax8(y4);
#pragma unroll
      for (int o = 8; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(FULL_MASK, amax, o));
      const float scale = fmaxf(__fdiv_rn(amax, 448.f), 1e-12f);
      *reinterpret_cast<uint2*>(xq_out + static_cast<size_t>(t) * H + c) = quant8_e4m3(y4, __fdiv_rn(1.f, scale));
      if ((tid & 15) == 0) xs_out[static_cast<size_t>(t) * (H / 128) + (c >> 7)] = scale;
    }
    return;
  }
  float gate = 0.f;
  if (!pad && gate_w != nullptr) {
    float dot = 0.f;
    for (int c = tid * 8; c < H; c += 2048) {
      const uint4 a = *reinterpret_cast<const uint4*>(x + static_cast<size_t>(t) * H + c);
      const uint4 w = *reinterpret_cast<const uint4*>(gate_w + c);
      dot = fmaf(bf_lo(a.x), bf_lo(w.x), dot); dot = fmaf(bf_hi(a.x), bf_hi(w.x), dot);
      dot = fmaf(bf_lo(a.y), bf_lo(w.y), dot); dot = fmaf(bf_hi(a.y), bf_hi(w.y), dot);
      dot = fmaf(bf_lo(a.z), bf_lo(w.z), dot); dot = fmaf(bf_hi(a.z), bf_hi(w.z), dot);
      dot = fmaf(bf_lo(a.w), bf_lo(w.w), dot); dot = fmaf(bf_hi(a.w), bf_hi(w.w), dot);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) dot += __shfl_xor_sync(FULL_MASK, dot, o);
    if ((tid & 31) == 0) red[tid >> 5] = dot;
    __syncthreads();
    float s = 0.f;
    for (int w = 0; w < 8; ++w) s += red[w];
    gate = 1.f / (1.f + __expf(-s));
  }
  float ss = 0.f;
  for (int c = tid * 8; c < H; c += 2048) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    if (!pad) {
      for (int j = 0; j < K; ++j) {
        const uint4 v = *reinterpret_cast<const uint4*>(cache + (static_cast<size_t>(t) * K + j) * H + c);
        acc[0] += bf_lo(v.x); acc[1] += bf_hi(v.x); acc[2] += bf_lo(v.y); acc[3] += bf_hi(v.y);
        acc[4] += bf_lo(v.z); acc[5] += bf_hi(v.z); acc[6] += bf_lo(v.w); acc[7] += bf_hi(v.w);
      }
      if (gate_w != nullptr) {
        const uint4 v = *reinterpret_cast<const uint4*>(cache + (static_cast<size_t>(T) * K + t) * H + c);
        acc[0] += gate * bf_lo(v.x); acc[1] += gate * bf_hi(v.x); acc[2] += gate * bf_lo(v.y); acc[3] += gate * bf_hi(v.y);
        acc[4] += gate * bf_lo(v.z); acc[5] += gate * bf_hi(v.z); acc[6] += gate * bf_lo(v.w); acc[7] += gate * bf_hi(v.w);
      }
    }
    const uint4 o4 = make_uint4(pack_bf2(acc[0], acc[1]), pack_bf2(acc[2], acc[3]), pack_bf2(acc[4], acc[5]),
                                pack_bf2(acc[6], acc[7]));
    if (out != nullptr) *reinterpret_cast<uint4*>(out + static_cast<size_t>(t) * H + c) = o4;
    const uint4 b = *reinterpret_cast<const uint4*>(residual + static_cast<size_t>(t) * H + c);
    float r[8] = {rbf(bf_lo(o4.x) + bf_lo(b.x)), rbf(bf_hi(o4.x) + bf_hi(b.x)), rbf(bf_lo(o4.y) + bf_lo(b.y)),
                  rbf(bf_hi(o4.y) + bf_hi(b.y)), rbf(bf_lo(o4.z) + bf_lo(b.z)), rbf(bf_hi(o4.z) + bf_hi(b.z)),
                  rbf(bf_lo(o4.w) + bf_lo(b.w)), rbf(bf_hi(o4.w) + bf_hi(b.w))};
#pragma unroll
    for (int i = 0; i < 8; ++i) ss = fmaf(r[i], r[i], ss);
    *reinterpret_cast<uint4*>(residual + static_cast<size_t>(t) * H + c) =
        make_uint4(pack_bf2(r[0], r[1]), pack_bf2(r[2], r[3]), pack_bf2(r[4], r[5]), pack_bf2(r[6], r[7]));
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(FULL_MASK, ss, o);
  if ((tid & 31) == 0) red2[tid >> 5] = ss;
  __syncthreads();
  float tot = 0.f;
  for (int i = 0; i < 8; ++i) tot += red2[i];
  const float rstd = rsqrtf(tot / H + eps);
  for (int c = tid * 8; c < H; c += 2048) {  // each thread re-reads the rows it wrote itself
    const uint4 b = *reinterpret_cast<const uint4*>(residual + static_cast<size_t>(t) * H + c);
    const uint4 g = *reinterpret_cast<const uint4*>(norm_w + c);
    const float r[8] = {bf_lo(b.x), bf_hi(b.x), bf_lo(b.y), bf_hi(b.y), bf_lo(b.z), bf_hi(b.z), bf_lo(b.w), bf_hi(b.w)};
    const float gw[8] = {bf_lo(g.x), bf_hi(g.x), bf_lo(g.y), bf_hi(g.y), bf_lo(g.z), bf_hi(g.z), bf_lo(g.w), bf_hi(g.w)};
    float y[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) y[i] = r[i] * rstd * (1.f + gw[i]);
    *reinterpret_cast<uint4*>(normed + static_cast<size_t>(t) * H + c) =
        make_uint4(pack_bf2(y[0], y[1]), pack_bf2(y[2], y[3]), pack_bf2(y[4], y[5]), pack_bf2(y[6], y[7]));
  }
}

// Expert-parallel dispatch: this rank's token rows and routing go straight into every rank's gathered buffers
// (its own included) with ordinary stores over NVLink; a barrier among the ranks follows on the host side.
// grid (world, 32): blockIdx.x = destination rank.
struct EpPushArgs {
  const uint4* x;        // [T_local, H] bf16 as 16-byte words
  const int32_t* ids;    // [T_local, K]
  const float* wts;      // [T_local, K]
  uint4* dst_x[8];       // rank r's x_all   [world * T_local, H]
  int32_t* dst_ids[8];   // rank r's ids_all [world * T_local, K]
  float* dst_wts[8];     // rank r's wts_all [world * T_local, K]
  int rank, x_words, route_n;  // 16-byte words of x, elements of ids / wts
};
__global__ void __launch_bounds__(256) ep_push_kernel(const EpPushArgs a) {
  pdl_wait();
  pdl_launch();
  const int d = blockIdx.x;
  uint4* dx = a.dst_x[d] + static_cast<size_t>(a.rank) * a.x_words;
  for (int i = blockIdx.y * 256 + threadIdx.x; i < a.x_words; i += gridDim.y * 256) dx[i] = a.x[i];
  if (blockIdx.y == 0) {
    int32_t* di = a.dst_ids[d] + static_cast<size_t>(a.rank) * a.route_n;
    float* dw = a.dst_wts[d] + static_cast<size_t>(a.rank) * a.route_n;
    for (int i = threadIdx.x; i < a.route_n; i += 256) {
      di[i] = a.ids[i];
      dw[i] = a.wts[i];
    }
  }
}

// workspace layout of the int8 block (all offsets 1024-byte aligned)
struct W8Layout {
  size_t xq, xs, h, hq, hs, total;
};
static W8Layout w8_layout(int T, int H, int I, int K) {
  const size_t rows = static_cast<size_t>(T) * (K + 1);
  auto up = [](size_t v) { return (v + 1023) & ~size_t(1023); };
  W8Layout l;
  size_t o = 0;
  l.xq = o; o = up(o + rows * H);
  l.xs = o; o = up(o + rows * 4);
  l.h = o;  o = up(o + rows * I * 2);
  l.hq = o; o = up(o + rows * I);
  l.hs = o; o = up(o + rows * 4);
  l.total = o;
  return l;
}

}  // namespace b200

using namespace b200;

extern "C" size_t b200_moe_w8a8_workspace_bytes(int T, int H, int I, int K) {
  if (T <= 0 || H <= 0 || I <= 0 || K <= 0) return 0;
  return w8_layout(T, H, I, K).total;
}

static int moe_w8a8_impl(const void* x, int T, int H, int I, int K, int E_local, const b200_moe_weights* w,
                         const b200_moe_lists* lists, void* cache, void* ws, size_t ws_bytes, int32_t* dbg_acc13,
                         void* dbg_h, int stages, int32_t* status, void* stream, void* const* peer_cache,
                         int ep_world, int ep_tokens_per_rank);

extern "C" int b200_moe_w8a8(const void* x, int T, int H, int I, int K, int E_local, const b200_moe_weights* w,
                             const b200_moe_lists* lists, void* cache, void* ws, size_t ws_bytes,
                             int32_t* dbg_acc13, void* dbg_h, int stages, int32_t* status, void* stream) {
  return moe_w8a8_impl(x, T, H, I, K, E_local, w, lists, cache, ws, ws_bytes, dbg_acc13, dbg_h, stages, status, stream,
                       nullptr, 0, 0);
}

extern "C" int b200_moe_w8a8_ep(const void* x, int T, int H, int I, int K, int E_local, const b200_moe_weights* w,
                                const b200_moe_lists* lists, void* const* peer_cache_host, int ep_world, int ep_rank,
                                int ep_tokens_per_rank, void* ws, size_t ws_bytes, int32_t* status, void* stream) {
  if (!peer_cache_host || ep_world < 1 || ep_world > 8 || ep_rank < 0 || ep_rank >= ep_world || ep_tokens_per_rank <= 0 ||
      T != ep_world * ep_tokens_per_rank)
    return fail(B200_E_ARG, "b200_moe_w8a8_ep: need 1 <= ep_world <= 8, 0 <= ep_rank < ep_world and T == ep_world * "
                "ep_tokens_per_rank (T=%d)", T);
  for (int r = 0; r < ep_world; ++r)
    if (!peer_cache_host[r] || (reinterpret_cast<uintptr_t>(peer_cache_host[r]) & 15))
      return fail(B200_E_ARG, "b200_moe_w8a8_ep: peer cache %d is null or not 16-byte aligned", r);
  return moe_w8a8_impl(x, T, H, I, K, E_local, w, lists, peer_cache_host[0], ws, ws_bytes, nullptr, nullptr, 0, status,
                       stream, peer_cache_host, ep_world | (ep_rank << 8), ep_tokens_per_rank);
}

static int moe_w8a8_impl(const void* x, int T, int H, int I, int K, int E_local, const b200_moe_weights* w,
                         const b200_moe_lists* lists, void* cache, void* ws, size_t ws_bytes, int32_t* dbg_acc13,
                         void* dbg_h, int stages, int32_t* status, void* stream, void* const* peer_cache,
                         int ep_world, int ep_tokens_per_rank) {
  if (!x || !w || !lists || !cache || !ws || !w->w13 || !w->s13 || !w->w2 || !w->s2)
    return fail(B200_E_ARG, "b200_moe_w8a8: null pointer");
  if (T <= 0 || K <= 0 || K > 32 || E_local <= 0 || H % 256 || I % 128 || H <= 0 || I <= 0)
    return fail(B200_E_ARG, "b200_moe_w8a8: need H %% 256 == 0, I %% 128 == 0, 1 <= K <= 32 (T=%d H=%d I=%d K=%d)", T, H,
                I, K);
  const W8Layout l = w8_layout(T, H, I, K);
  if (ws_bytes < l.total) return fail(B200_E_WS, "b200_moe_w8a8: workspace %zu < %zu bytes", ws_bytes, l.total);
  if (reinterpret_cast<uintptr_t>(ws) & 1023) return fail(B200_E_ALIGN, "b200_moe_w8a8: workspace must be 1024-byte aligned");
  if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(cache)) & 15)
    return fail(B200_E_ALIGN, "b200_moe_w8a8: x and cache must be 16-byte aligned");
  const bool shared = w->sh13 != nullptr;
  if (shared && (!w->shs13 || !w->sh2 || !w->shs2)) return fail(B200_E_ARG, "b200_moe_w8a8: incomplete shared expert");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  uint8_t* base = static_cast<uint8_t*>(ws);
  int8_t* xq = reinterpret_cast<int8_t*>(base + l.xq);
  float* xs = reinterpret_cast<float*>(base + l.xs);
  bf16* h = reinterpret_cast<bf16*>(base + l.h);
  int8_t* hq = reinterpret_cast<int8_t*>(base + l.hq);
  float* hs = reinterpret_cast<float*>(base + l.hs);
  const int rows = T * (K + 1);
  MoeLists L{lists->counts,     lists->offsets,  lists->row_of_pair, lists->slot_of_row, lists->wt_of_row,
             lists->blk_expert, lists->blk_row0, lists->blk_rows,    lists->nblocks};

  CUtensorMap tmW13, tmSh13, tmXq, tmXq64, tmXq128, tmW2, tmSh2, tmHq, tmHq64, tmHq128;
  int rc;
  if ((rc = make_tmap_bytes_2d(&tmW13, w->w13, static_cast<uint64_t>(E_local) * 2 * I, H, 128, "w13"))) return rc;
  if ((rc = make_tmap_bytes_2d(&tmSh13, shared ? w->sh13 : w->w13, 2 * I, H, 128, "sh13"))) return rc;
  if ((rc = make_tmap_bytes_2d(&tmXq, xq, rows, H, 16, "xq"))) return rc;
  if ((rc = make_tmap_bytes_2d(&tmXq64, xq, rows, H, 64, "xq"))) return rc;
  if ((rc = make_tmap_bytes_2d(&tmXq128, xq, rows, H, 128, "xq"))) return rc;
  if ((rc = make_tmap_bytes_2d(&tmW2, w->w2, static_cast<uint64_t>(E_local) * H, I, 128, "w2"))) return rc;
  if ((rc = make_tmap_bytes_2d(&tmSh2, shared ? w->sh2 : w->w2, H, I, 128, "sh2"))) return rc;
  if ((rc = make_tmap_bytes_2d(&tmHq, hq, rows, I, 16, "hq"))) return rc;
  if ((rc = make_tmap_bytes_2d(&tmHq64, hq, rows, I, 64, "hq"))) return rc;
  if ((rc = make_tmap_bytes_2d(&tmHq128, hq, rows, I, 128, "hq"))) return rc;

  static DeviceOnce once;
  once.run([] {
    cudaFuncSetAttribute(moe_gemm_i8_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, GemmCfg<true>::SMEM);
    cudaFuncSetAttribute(moe_gemm_i8_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, GemmCfg<false>::SMEM);
  });

  if ((stages & 15) == 0) stages |= 15;
  // tokens that get a shared-expert row: all of them, or this rank's own under expert parallelism
  int shared_lo = 0, shared_n = T;
  if ((ep_world & 0xff) >= 1) {
    shared_lo = (ep_world >> 8) * ep_tokens_per_rank;
    shared_n = ep_tokens_per_rank;
  }
  if (stages & B200_MOE_STAGE_QUANT)
    launch_k(quant_permute_i8_kernel, dim3(T), dim3(256), 0, st, static_cast<const bf16*>(x), T, H, K, L.row_of_pair,
             shared_lo, shared ? shared_n : 0, xq, xs);

  GemmArgs a{};
  a.L = L;
  a.E_local = E_local;
  a.I = I;
  a.H = H;
  a.total_rows = rows;
  a.status = status;
  a.test_starve = (stages & B200_MOE_TEST_STARVE) ? 1 : 0;
  const int grid = sm_count();

  a.mtiles = I / 128;
  a.ksteps = H / 128;
  a.w_rows = 2 * I;
  a.s_w = w->s13;
  a.s_w_sh = w->shs13;
  a.a_scale = xs;
  a.h_out = h;
  a.dbg_acc = dbg_acc13;
  a.dbg_h = static_cast<bf16*>(dbg_h);
  if (stages & B200_MOE_STAGE_UP)
    // the kernel reads the routing lists before its dependency wait: only safe to start early when the kernel
    // right before it in the stream is this call's own quantiser (which itself waited for the lists)
    if (stages & B200_MOE_STAGE_QUANT)
      launch_k(moe_gemm_i8_kernel<true>, dim3(grid), dim3(GEMM_THREADS), GemmCfg<true>::SMEM, st, tmW13, tmSh13, tmXq,
               tmXq64, tmXq128, a);
    else
      moe_gemm_i8_kernel<true><<<grid, GEMM_THREADS, GemmCfg<true>::SMEM, st>>>(tmW13, tmSh13, tmXq, tmXq64, tmXq128, a);

  if (stages & B200_MOE_STAGE_HQUANT)
    launch_k(quant_rows_i8_kernel, dim3((rows + 7) / 8), dim3(256), 0, st, h, rows, I, L.slot_of_row, hq, hs);

  a.mtiles = H / 256;  // two consecutive 128-row tiles of W2 per GEMM tile: the token tile is read half as often
  a.ksteps = I / 128;
  a.w_rows = H;
  a.s_w = w->s2;
  a.s_w_sh = w->shs2;
  a.a_scale = hs;
  a.h_out = nullptr;
  a.cache = static_cast<bf16*>(cache);
  a.dbg_acc = nullptr;
  a.dbg_h = nullptr;
  a.ep_world = ep_world & 0xff;
  a.ep_rank = ep_world >> 8;
  a.ep_tokens = ep_tokens_per_rank;
  a.ep_rows = ep_tokens_per_rank * K;
  ep_world &= 0xff;
  for (int r = 0; r < 8; ++r) a.ep_cache[r] = (peer_cache && r < ep_world) ? static_cast<bf16*>(peer_cache[r]) : nullptr;
  if (stages & B200_MOE_STAGE_DOWN)
    if (stages & B200_MOE_STAGE_HQUANT)
      launch_k(moe_gemm_i8_kernel<false>, dim3(grid), dim3(GEMM_THREADS), GemmCfg<false>::SMEM, st, tmW2, tmSh2, tmHq,
               tmHq64, tmHq128, a);
    else
      moe_gemm_i8_kernel<false><<<grid, GEMM_THREADS, GemmCfg<false>::SMEM, st>>>(tmW2, tmSh2, tmHq, tmHq64, tmHq128, a);
  return launch_status("b200_moe_w8a8");
}

extern "C" int b200_moe_combine(const void* cache, const void* x, const void* gate_w, const int64_t* pos, int T, int H,
                                int K, void* out, void* stream) {
  if (!cache || !out || (gate_w && !x)) return fail(B200_E_ARG, "b200_moe_combine: null pointer");
  if (T < 0 || H <= 0 || H % 8 || K <= 0) return fail(B200_E_ARG, "b200_moe_combine: need H %% 8 == 0 (H=%d K=%d)", H, K);
  if (T == 0) return 0;
  launch_k(moe_combine_kernel, dim3(T), dim3(256), 0, static_cast<cudaStream_t>(stream), static_cast<const bf16*>(cache),
           static_cast<const bf16*>(x), static_cast<const bf16*>(gate_w), pos, T, H, K, static_cast<bf16*>(out));
  return launch_status("b200_moe_combine");
}

static int combine_norm_impl(const void* cache, const void* x, const void* gate_w, const int64_t* pos, int T, int H, int K,
                             void* out, void* residual, const void* norm_w, float eps, void* normed, void* xq_out,
                             float* xs_out, void* stream) {
  if (!cache || !x || !residual || !norm_w || !normed) return fail(B200_E_ARG, "b200_moe_combine_norm: null pointer");
  if (T < 0 || H <= 0 || H % 8 || K <= 0)
    return fail(B200_E_ARG, "b200_moe_combine_norm: need H %% 8 == 0 (H=%d K=%d)", H, K);
  if ((xq_out != nullptr) != (xs_out != nullptr) || (xq_out != nullptr && (H != 2048 || K > 12)))
    return fail(B200_E_ARG, "b200_moe_combine_norm_q: the quantised row needs both outputs, H == 2048 and K <= 12 (H=%d K=%d)",
                H, K);
  if (T == 0) return 0;
  launch_k(moe_combine_norm_kernel, dim3(T), dim3(256), 0, static_cast<cudaStream_t>(stream),
           static_cast<const bf16*>(cache), static_cast<const bf16*>(x), static_cast<const bf16*>(gate_w), pos, T, H, K,
           static_cast<bf16*>(out), static_cast<bf16*>(residual), static_cast<const bf16*>(norm_w), eps,
           static_cast<bf16*>(normed), static_cast<uint8_t*>(xq_out), xs_out);
  return launch_status("b200_moe_combine_norm");
}

extern "C" int b200_moe_combine_norm(const void* cache, const void* x, const void* gate_w, const int64_t* pos, int T, int H,
                                     int K, void* out, void* residual, const void* norm_w, float eps, void* normed,
                                     void* stream) {
  return combine_norm_impl(cache, x, gate_w, pos, T, H, K, out, residual, norm_w, eps, normed, nullptr, nullptr, stream);
}

extern "C" int b200_moe_combine_norm_q(const void* cache, const void* x, const void* gate_w, const int64_t* pos, int T,
                                       int H, int K, void* out, void* residual, const void* norm_w, float eps,
                                       void* normed, void* xq_out, float* xs_out, void* stream) {
  if (!xq_out || !xs_out) return fail(B200_E_ARG, "b200_moe_combine_norm_q: null pointer");
  return combine_norm_impl(cache, x, gate_w, pos, T, H, K, out, residual, norm_w, eps, normed, xq_out, xs_out, stream);
}

extern "C" int b200_ep_push(const void* x, const int32_t* ids, const float* wts, int T_local, int H, int K, int ep_rank,
                            int ep_world, void* const* peer_x_host, void* const* peer_ids_host,
                            void* const* peer_wts_host, void* stream) {
  if (!x || !ids || !wts || !peer_x_host || !peer_ids_host || !peer_wts_host)
    return fail(B200_E_ARG, "b200_ep_push: null pointer");
  if (T_local <= 0 || H <= 0 || H % 8 || K <= 0 || ep_world < 1 || ep_world > 8 || ep_rank < 0 || ep_rank >= ep_world)
    return fail(B200_E_ARG, "b200_ep_push: need H %% 8 == 0, 1 <= ep_world <= 8, 0 <= ep_rank < ep_world (H=%d world=%d)", H,
                ep_world);
  EpPushArgs a{};
  a.x = static_cast<const uint4*>(x);
  a.ids = ids;
  a.wts = wts;
  a.rank = ep_rank;
  a.x_words = T_local * (H / 8);
  a.route_n = T_local * K;
  for (int r = 0; r < ep_world; ++r) {
    if (!peer_x_host[r] || !peer_ids_host[r] || !peer_wts_host[r] || (reinterpret_cast<uintptr_t>(peer_x_host[r]) & 15))
      return fail(B200_E_ALIGN, "b200_ep_push: rank %d's buffers must be non-null and 16-byte aligned", r);
    a.dst_x[r] = static_cast<uint4*>(peer_x_host[r]);
    a.dst_ids[r] = static_cast<int32_t*>(peer_ids_host[r]);
    a.dst_wts[r] = static_cast<float*>(peer_wts_host[r]);
  }
  if (reinterpret_cast<uintptr_t>(x) & 15) return fail(B200_E_ALIGN, "b200_ep_push: x must be 16-byte aligned");
  launch_k(ep_push_kernel, dim3(ep_world, 32), dim3(256), 0, static_cast<cudaStream_t>(stream), a);
  return launch_status("b200_ep_push");
}
