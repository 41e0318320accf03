// MoE block in fp8 e4m3 with 128 x 128 weight block scales and per-(token, 128-channel) activation
// scales: activation quantise + permute, grouped GEMMs on tcgen05 (kind::f8f6f4), SwiGLU / unpermute
// epilogues.  The reference has no block-scaled fp8 MoE; the structure follows its int8 twin
// (qk_moe_prefill_i8.cu:3649-3651, 3905-3945): per 128-k block the MMA chain starts from zero in a
// TMEM partial buffer and is promoted by the epilogue warps, acc = fma(partial, a_scale * w_scale,
// acc).  All 512 TMEM columns are partial buffers (8 of 64 columns: 2 x 32 in the expert GEMMs, whose blocks have at
// most 32 rows; 4 of 128 in the dense modes over 128-row chunks), so the MMA issuer runs up to eight k blocks ahead
// of the promotion warps, which also run the epilogue: a tile's epilogue no longer stalls the weight stream.
//
// Orientation as in the int8 kernels: M = 128 weight rows (exactly one weight scale block row),
// N = 16 or 32 tokens of one expert (16..128 rows of a chunk in the dense modes), K = 32 bytes per MMA; weights and
// expert-sorted token rows arrive by 2-D TMA with the 128-byte swizzle.  Final accumulators live in registers
// (16 + 16 fp32 per thread for the two weight tiles of a stage; 32 in the dense modes).
#include "common.cuh"
#include "host.h"

namespace b200 {

B200_DEFINE_WAIT_BUDGET_SETTER(set_wait_budget_moe_fp8)

constexpr int F8_TILE = 128 * 128;       // weight tile bytes per stage
constexpr int F8_BTILE = 64 * 128;       // token tile bytes per stage, dense modes (<= 64 rows)
constexpr int F8_BTILE_MOE = 32 * 128;   // the same in the expert GEMMs (blocks of <= 32 rows)
constexpr int F8_THREADS = 320;          // TMA warp, MMA warp, 8 epilogue warps (two per TMEM lane quadrant)
constexpr int F8_THREADS_WIDE = 576;     // the same with 16 epilogue warps (four per quadrant, 32 columns each)
constexpr int F8_CACHED = 1024;          // blocks of the list whose entries every CTA of a MoE GEMM keeps in shared memory
constexpr int F8_MAXKG = 32;             // k blocks per row of scales held in shared memory (K <= 4096)
constexpr int F8_WS_FLOATS = 1024;       // weight block scales of the CTA's first tiles, cached in shared memory

// ---- activation quantisers (quant8_e4m3 / amax8: common.cuh) ----
// How the expert GEMMs cut their tile sequence over the CTAs: tile = (block, weight tile), weight tile fastest; a tile
// costs cost_base + 16-row units of its block; CTA j of `grid` takes the tiles whose cost interval starts in
// [total j / grid, total (j + 1) / grid).  The table of the grid + 1 boundaries is computed once per call by one extra
// CTA of the activation quantiser's launch, for the gate/up GEMM (table 0) and the down GEMM (table 1), so that a GEMM CTA
// starts streaming after two short round trips to memory instead of caching and scanning the whole block list (4.9 us
// before the first load at 516 blocks).  table[0] = -1: no table (more than F8_CACHED blocks).
struct F8Partition {
  const int32_t* blk_rows;
  const int32_t* nblocks;
  int grid;
  int mtiles[2], cost_base[2];
  int32_t* table[2];   // [grid + 1] each
};
constexpr int F8_PART_INTS = 160;   // room for grid + 1 boundaries (148 SMs)

__device__ void f8_partition_tiles(const F8Partition& q) {
  __shared__ int cpre[2][F8_CACHED + 1];
  __shared__ int wsum[2][8];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int nblocks = q.nblocks[0];
  if (nblocks > F8_CACHED || nblocks < 0 || q.grid + 1 > F8_PART_INTS) {
    if (tid == 0) q.table[0][0] = q.table[1][0] = -1;
    return;
  }
  // thread t owns blocks [4 t, 4 t + 4): F8_CACHED = 4 x 256
  int nb16[4], sum[2] = {0, 0};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int b = 4 * tid + i;
    nb16[i] = b < nblocks ? (q.blk_rows[b] + 15) >> 4 : -1;
    if (nb16[i] >= 0) {
      sum[0] += q.mtiles[0] * (q.cost_base[0] + nb16[i]);
      sum[1] += q.mtiles[1] * (q.cost_base[1] + nb16[i]);
    }
  }
  int incl[2] = {sum[0], sum[1]};
#pragma unroll
  for (int o = 1; o < 32; o <<= 1)
#pragma unroll
    for (int g = 0; g < 2; ++g) {
      const int v = __shfl_up_sync(FULL_MASK, incl[g], o);
      if (lane >= o) incl[g] += v;
    }
  if (lane == 31) {
    wsum[0][warp] = incl[0];
    wsum[1][warp] = incl[1];
  }
  __syncthreads();
#pragma unroll
  for (int g = 0; g < 2; ++g) {
    int run = incl[g] - sum[g];
    for (int w = 0; w < warp; ++w) run += wsum[g][w];
#pragma unroll
    for (int i = 0; i < 4; ++i)
      if (nb16[i] >= 0) {
        cpre[g][4 * tid + i] = run;
        run += q.mtiles[g] * (q.cost_base[g] + nb16[i]);
      }
    if (4 * tid < nblocks && 4 * tid + 4 >= nblocks) cpre[g][nblocks] = run;   // the owner of the last block
  }
  __syncthreads();
  for (int j = tid; j <= q.grid; j += 256)
#pragma unroll
    for (int g = 0; g < 2; ++g) {
      const int ntiles = nblocks * q.mtiles[g];
      const long long total = nblocks > 0 ? cpre[g][nblocks] : 0;
      const long long c = total * j / q.grid;
      int at = ntiles;
      if (j == 0) {
        at = 0;
      } else if (j < q.grid && c < total) {
        int lo = 0, hi = nblocks - 1;   // last block with cpre[blk] <= c
        while (lo < hi) {
          const int mid = (lo + hi + 1) >> 1;
          if (cpre[g][mid] <= c) lo = mid; else hi = mid - 1;
        }
        const int tc = (cpre[g][lo + 1] - cpre[g][lo]) / q.mtiles[g];
        int within = static_cast<int>((c - cpre[g][lo]) / tc);
        if (within >= q.mtiles[g]) within = q.mtiles[g] - 1;
        at = lo * q.mtiles[g] + within;
      }
      q.table[g][j] = at;
    }
}

// one CTA per token; 16 consecutive threads own one 128-channel group (8 channels each)
// tokens [shared_lo, shared_lo + shared_n) also get their shared-expert row T*K + t
__global__ void __launch_bounds__(256) quant_permute_f8_kernel(const bf16* __restrict__ x, int T, int H, int K,
                                                               const int32_t* __restrict__ row_of_pair,
                                                               int shared_lo, int shared_n, uint8_t* __restrict__ xq,
                                                               float* __restrict__ xs, const F8Partition part) {
  __shared__ int rows[40];
  const int t = blockIdx.x, tid = threadIdx.x;
  if (t == T) {   // the extra CTA of the expert block's launch: tile boundaries of the two GEMMs that follow
    f8_partition_tiles(part);
    return;
  }
  if (tid < K) rows[tid] = row_of_pair[t * K + tid];
  if (tid == K) rows[K] = (t >= shared_lo && t < shared_lo + shared_n) ? T * K + t : -1;
  __syncthreads();
  const int KG = H / 128;
  for (int c = tid * 8; c < H; c += 2048) {
    const uint4 v = *reinterpret_cast<const uint4*>(x + static_cast<size_t>(t) * H + c);
    float amax = amax8(v);
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(FULL_MASK, amax, o));
    const float scale = fmaxf(__fdiv_rn(amax, 448.f), 1e-12f);
    const uint2 q = quant8_e4m3(v, __fdiv_rn(1.f, scale));
    for (int j = 0; j <= K; ++j) {
      const int row = rows[j];
      if (row >= 0) {
        *reinterpret_cast<uint2*>(xq + static_cast<size_t>(row) * H + c) = q;
        if ((tid & 15) == 0) xs[static_cast<size_t>(row) * KG + (c >> 7)] = scale;
      }
    }
  }
}

// h bf16 [rows, I] -> e4m3 + scale per (row, 128 channels); one warp per sorted row
__global__ void __launch_bounds__(256) quant_rows_f8_kernel(const bf16* __restrict__ h, int rows, int I,
                                                            const int32_t* __restrict__ slot_of_row,
                                                            uint8_t* __restrict__ hq, float* __restrict__ hs) {
  const int row = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (row >= rows || slot_of_row[row] < 0) return;
  const int KG = I / 128;
  for (int c = lane * 8; c < I; c += 256) {
    const uint4 v = *reinterpret_cast<const uint4*>(h + static_cast<size_t>(row) * I + c);
    float amax = amax8(v);
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(FULL_MASK, amax, o));
    const float scale = fmaxf(__fdiv_rn(amax, 448.f), 1e-12f);
    *reinterpret_cast<uint2*>(hq + static_cast<size_t>(row) * I + c) = quant8_e4m3(v, __fdiv_rn(1.f, scale));
    if ((lane & 15) == 0) hs[static_cast<size_t>(row) * KG + (c >> 7)] = scale;
  }
}

// ---- grouped fp8 GEMM -------------------------------------------------------------------------------------
struct F8Args {
  MoeLists L;
  int E_local, mtiles, ksteps, w_rows, I, H, total_rows;
  const float* s_w;      // routed weight block scales [E_local, w_rows/128, ksteps]
  const float* s_w_sh;   // shared expert [w_rows/128, ksteps]
  const float* a_scale;  // [total_rows, ksteps]
  bf16* h_out;           // up: sorted rows [total_rows, I]
  bf16* cache;           // down: [total_rows, H] by slot
  bf16* dbg_h;           // up: h by slot or null
  int32_t* status;
  // LM-head mode: one dense block of `total_rows` tokens against w_rows vocabulary rows
  unsigned long long* lm_keys;  // [mtiles * 4][total_rows] packed (value, id) maxima, one row per (tile, warp)
  float* lm_logits;             // [total_rows, w_rows] or null
  int lm_shard_lo;
  int lm_ld;                    // row pitch of lm_logits (elements)
  // dense mode: output features [seg_lo[i], seg_lo[i+1]) go to seg_out[i] with row pitch seg_ld[i]; boundaries
  // are multiples of 32, so the 32 features of a warp share one segment
  int nseg;
  int seg_lo[5];
  int seg_ld[4];
  bf16* seg_out[4];
  // expert-parallel down epilogue: routed slot s of the gathered batch belongs to rank s / ep_rows, whose cache
  // (this GPU's own, or a peer's mapped over NVLink) receives the row at local slot s % ep_rows; shared-expert
  // rows are kept only for this rank's own tokens
  int ep_world;                 // 0: single GPU, rows go to `cache`
  int ep_rows, ep_rank, ep_tokens;
  bf16* ep_cache[8];
  int test_starve;  // self-test: the producer leaves out the token rows, so no stage ever completes and every wait runs out
  int cost_base;    // cost of a tile in 16-row units of tokens, before its token rows are counted (tile partition)
  // dense mode with partial sums: the K range is cut into `kparts` equal parts whose fp32 sums (each a promotion
  // chain from zero) go to partials[part][row][feature]; the consumer adds the parts in part order, so the
  // arithmetic is fixed by `kparts` alone.  A tile covers kparts / ksplit consecutive parts: `ksplit` only says over
  // how many CTAs the K range of one (weight tile, row chunk) is spread (1: bf16 outputs when partials is null).
  int ksplit, kparts;
  float* partials;
  const int32_t* part;   // expert GEMMs: this launch's tile boundaries [grid + 1] (F8Partition), or null
};

constexpr int MODE_DOWN = 0, MODE_UP = 1, MODE_LM = 2, MODE_DENSE = 3;
// The dense modes over 128-row chunks of the token rows (more than 64 rows in the call): the weight tile is read half
// as often per row, and every activation scale of the call sits in shared memory from the start.
constexpr int MODE_DENSE_W = 4, MODE_LM_W = 5;
constexpr int F8_AS_FLOATS = 8192;       // wide modes: activation scales [k blocks][rows padded to 128]

template <int MODE>
struct F8Cfg {
  static constexpr bool UP = MODE == MODE_UP;
  // two weight tiles per stage against one token tile: gate + up rows of one channel block (up), two consecutive
  // 128-row tiles of W2 (down: the token tile is read half as often and every per-tile cost is paid half as often)
  static constexpr bool DUAL = MODE == MODE_UP || MODE == MODE_DOWN;
  static constexpr bool WIDE = MODE == MODE_DENSE_W || MODE == MODE_LM_W;
  static constexpr int NA = DUAL ? 2 : 1;
  static constexpr int STAGE = NA * F8_TILE + (WIDE ? F8_TILE : DUAL ? F8_BTILE_MOE : F8_BTILE);
  static constexpr int STAGES = WIDE ? 5 : (DUAL ? 5 : 7);
  // TMEM columns of one partial buffer.  The expert GEMMs take blocks of at most 32 rows, so a partial is 2 x 32
  // columns and eight of them fit: the MMA issuer runs up to eight k blocks ahead of the promotion, which covers a
  // tile's epilogue (and two whole tiles of the down GEMM).
  static constexpr int PW = WIDE ? 128 : 64;
  static constexpr int NPB = 512 / PW;       // partial buffers
  static constexpr int NL = DUAL ? 16 : 32;  // columns (token rows) of a tile that one epilogue warp owns
  static constexpr int THREADS = WIDE ? F8_THREADS_WIDE : F8_THREADS;
  static constexpr int EPI_WARPS = (THREADS - 64) / 32;
  static constexpr int META_WARP = (WIDE ? 0 : NL * F8_MAXKG * 4) + 32 * 8 + 2 * F8_MAXKG * 4;
  static constexpr int META = EPI_WARPS * META_WARP;  // per epilogue warp: activation scales, slot, weight of its 32 columns, weight scales
  static constexpr bool LISTS = MODE == MODE_UP || MODE == MODE_DOWN;
  static constexpr int TINFO = LISTS ? F8_CACHED * 12 + (F8_CACHED + 32) * 4 : 64;  // block entries + cost prefix
  static constexpr int SMEM = STAGES * STAGE + 1024 + 256 + META + TINFO + F8_WS_FLOATS * 4 + (WIDE ? F8_AS_FLOATS * 4 : 0);
  static constexpr int TMEM = 512;
};

// Optional timeline of CTA 0 (compile with -DB200_TRACE): %globaltimer stamps of the producer's TMA issues (row 0),
// the MMA issuer's stage arrivals (row 1), the first epilogue warp's promotions (row 2) and tile boundaries (row 3).
#ifdef B200_TRACE
__device__ unsigned long long g_trace[6][256];
__device__ unsigned long long g_cta[256][4];
#define TRACE(k, i) do { if (blockIdx.x == 0 && (i) < 256) g_trace[k][i] = globaltimer(); } while (0)
#else
#define TRACE(k, i) do { } while (0)
#endif

template <int MODE>
__global__ void __launch_bounds__(F8Cfg<MODE>::THREADS, 1)
moe_gemm_f8_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmWsh,
                   const __grid_constant__ CUtensorMap tmX, const __grid_constant__ CUtensorMap tmX64, const F8Args p) {
  using C = F8Cfg<MODE>;
  constexpr bool UP = MODE == MODE_UP, DENSE = MODE == MODE_DENSE || MODE == MODE_DENSE_W;
  constexpr bool LM = MODE == MODE_LM || MODE == MODE_LM_W || DENSE;   // no lists: blocks are chunks of the token rows
  constexpr bool DUAL = C::DUAL, WIDE = C::WIDE;
  constexpr int NL = C::NL, NH2 = DUAL ? 1 : 2;
  constexpr int BROWS = DUAL ? 32 : 64;   // most rows of a block
  constexpr int CH = WIDE ? 128 : 64;   // token rows of a chunk in the dense modes
  constexpr int MROWS = (MODE == MODE_DOWN) ? 256 : 128;  // weight rows (output features) per tile
  // second weight tile of a stage: the up rows of the same channels (I rows further), or the next 128 rows of W2
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + C::STAGES * C::STAGE);
  uint64_t* empty = full + C::STAGES;
  uint64_t* pfull = empty + C::STAGES;   // [NPB] a 128-k partial is complete in TMEM
  uint64_t* pempty = pfull + C::NPB;     // [NPB] the epilogue warps have promoted it
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(pempty + C::NPB);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  uint8_t* meta = smem + C::STAGES * C::STAGE + 256;
  int* tinfo = reinterpret_cast<int*>(meta + C::META);   // [F8_CACHED][3] expert, first row, rows of each block
  int* cprefix = tinfo + F8_CACHED * 3;                  // [F8_CACHED + 1] cost of the blocks before each block
  float* ws_cache = reinterpret_cast<float*>(meta + C::META + C::TINFO);
  float* as_all = ws_cache + F8_WS_FLOATS;               // wide modes: [ksteps][tpad]

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int s = 0; s < C::STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int b = 0; b < C::NPB; ++b) {
      mbar_init(&pfull[b], 1);
      mbar_init(&pempty[b], C::EPI_WARPS);
    }
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmW);
    tma_prefetch_desc(&tmWsh);
    tma_prefetch_desc(&tmX);
    tma_prefetch_desc(&tmX64);
  }
  if (warp == 1) tmem_alloc(tmem_slot, C::TMEM);   // its latency hides behind the list reads below
  // Tiles are (block, weight tile) pairs, weight tile fastest; each CTA takes a contiguous range, so consecutive
  // tiles mostly share their block and its metadata.  Every CTA reads the whole block list into shared memory
  // before the weight stream starts (afterwards a dependent global load costs microseconds: it queues behind
  // the stages in flight) and cuts the tile sequence by COST, not by count: a tile with many token rows takes
  // longer (more token bytes, more accumulator columns to promote), and the blocks of one expert, the shared
  // expert above all, are neighbours in the list, so equal counts would hand one CTA all the heavy tiles.
  // (The dense modes have no lists: their blocks are the 64- or 128-row chunks of the token rows, and a tile is
  // (weight tile, chunk) with the chunk fastest, so the chunks of one weight tile run back to back on one CTA
  // and all but the first find the weight tile in L2.)
  const int nblocks = LM ? (p.total_rows + CH - 1) / CH : p.L.nblocks[0];
  const int tpad = nblocks * 128;
  const int ntiles = nblocks * p.mtiles * (DENSE ? p.ksplit : 1);
  int t_lo = static_cast<int>(static_cast<long long>(blockIdx.x) * ntiles / gridDim.x);
  int t_hi = static_cast<int>(static_cast<long long>(blockIdx.x + 1) * ntiles / gridDim.x);
  auto blk_of = [&](int tile) { return LM ? tile % nblocks : tile / p.mtiles; };
  // k blocks of one tile and the first of them (split-K in the dense mode; the whole K otherwise)
  const int kn = DENSE ? p.ksteps / p.ksplit : p.ksteps;
  auto k0_of = [&](int tile) { return DENSE ? ((tile / nblocks) % p.ksplit) * kn : 0; };
  bool have_part = false;
  if (C::LISTS && p.part != nullptr) {
    // boundaries computed by the quantiser launch of this call: only this CTA's own blocks are cached
    const int lo = p.part[blockIdx.x], hi = p.part[blockIdx.x + 1];
    if (p.part[0] == 0 && lo >= 0 && lo <= hi && hi <= ntiles && (blockIdx.x + 1 < gridDim.x || hi == ntiles)) {
      have_part = true;
      t_lo = lo;
      t_hi = hi;
      const int b_lo = lo / p.mtiles, b_hi = hi > lo ? (hi - 1) / p.mtiles : b_lo - 1;
      for (int blk = b_lo + static_cast<int>(threadIdx.x); blk <= b_hi && blk < F8_CACHED; blk += C::THREADS) {
        tinfo[blk * 3 + 0] = p.L.blk_expert[blk];
        tinfo[blk * 3 + 1] = p.L.blk_row0[blk];
        tinfo[blk * 3 + 2] = p.L.blk_rows[blk];
      }
    }
  }
  if (C::LISTS && !have_part) {
    const int ncached = nblocks < F8_CACHED ? nblocks : F8_CACHED;
    for (int blk = threadIdx.x; blk < ncached; blk += C::THREADS) {
      tinfo[blk * 3 + 0] = p.L.blk_expert[blk];
      tinfo[blk * 3 + 1] = p.L.blk_row0[blk];
      tinfo[blk * 3 + 2] = p.L.blk_rows[blk];
    }
    __syncthreads();
    if (nblocks <= F8_CACHED) {
      // cost of a tile = cost_base + 16-row units of its block; prefix over the blocks by warp 0
      if (warp == 0) {
        const int chunk = (nblocks + 31) / 32, lo = lane * chunk, hi = lo + chunk < nblocks ? lo + chunk : nblocks;
        int sum = 0;
        for (int b = lo; b < hi; ++b) sum += p.mtiles * (p.cost_base + ((tinfo[b * 3 + 2] + 15) >> 4));
        int incl = sum;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
          const int v = __shfl_up_sync(FULL_MASK, incl, o);
          if (lane >= o) incl += v;
        }
        int run = incl - sum;
        for (int b = lo; b < hi; ++b) {
          cprefix[b] = run;
          run += p.mtiles * (p.cost_base + ((tinfo[b * 3 + 2] + 15) >> 4));
        }
        if (lane == 31) cprefix[nblocks] = incl;
      }
      __syncthreads();
      const long long total = cprefix[nblocks];
      auto tile_at = [&](long long c) -> int {   // first tile whose cost interval ends after cost position c
        if (c >= total) return ntiles;
        int lo = 0, hi = nblocks - 1;            // last block with cprefix[blk] <= c
        while (lo < hi) {
          const int mid = (lo + hi + 1) >> 1;
          if (cprefix[mid] <= c) lo = mid; else hi = mid - 1;
        }
        const int tc = p.cost_base + ((tinfo[lo * 3 + 2] + 15) >> 4);
        int within = static_cast<int>((c - cprefix[lo]) / tc);
        if (within >= p.mtiles) within = p.mtiles - 1;
        return lo * p.mtiles + within;
      };
      t_lo = blockIdx.x == 0 ? 0 : tile_at(total * blockIdx.x / gridDim.x);
      t_hi = blockIdx.x + 1 == gridDim.x ? ntiles : tile_at(total * (blockIdx.x + 1) / gridDim.x);
    }
  }
  __syncthreads();

  auto decode = [&](int tile, int& e, int& row0, int& n, int& mt) -> bool {
    if (LM) {  // dense: 128 weight rows against one chunk of the token rows (and one part of K when split)
      e = 0;
      const int mx = tile / nblocks;
      mt = DENSE ? mx / p.ksplit : mx;
      row0 = (tile - mx * nblocks) * CH;
      n = p.total_rows - row0 < CH ? p.total_rows - row0 : CH;
      return n >= 1;
    }
    const int blk = tile / p.mtiles;
    mt = tile - blk * p.mtiles;
    if (blk < F8_CACHED) {
      e = tinfo[blk * 3 + 0];
      row0 = tinfo[blk * 3 + 1];
      n = tinfo[blk * 3 + 2];
    } else {
      e = p.L.blk_expert[blk];
      row0 = p.L.blk_row0[blk];
      n = p.L.blk_rows[blk];
    }
    return e >= 0 && e <= p.E_local && n >= 1 && n <= BROWS && row0 >= 0 && row0 + n <= p.total_rows;
  };

  // Per-block metadata of an epilogue warp (activation scales, slot and routing weight of its 32 columns) is
  // loaded into registers one block ahead: the loads for the next block are issued when a block's first
  // tile starts and are consumed at the next block's first tile; the first block's loads are issued
  // before the producer starts.  Weight block scales are loaded two tiles ahead.  No loaded value is
  // consumed where it is fetched.
  struct Meta {
    float v[16];
    float wt;
    int slot;
  };
  const int ep_half = (warp - 2) >> 2;
  // tile column of an epilogue warp's local column l: the two warps of a lane quadrant take alternate 16-column chunks
  auto col_of = [&](int l) {
    return DUAL ? ep_half * 16 + l : WIDE ? ep_half * 32 + l : (l >> 4) * 32 + ep_half * 16 + (l & 15);
  };
  auto fetch = [&](int tile, Meta& m) {  // the metadata of the block that `tile` belongs to
    m.wt = 0.f;
    m.slot = -1;
#pragma unroll
    for (int u = 0; u < 16; ++u) m.v[u] = 0.f;
    int e, row0, n, mt;
    if (WIDE || tile >= t_hi || !decode(tile, e, row0, n, mt)) return;
    const int c = col_of(lane);
    if (!LM && lane < NL && c < n) {
      m.slot = p.L.slot_of_row[row0 + c];
      m.wt = p.L.wt_of_row[row0 + c];
    }
    const int total = NL * p.ksteps;
#pragma unroll
    for (int u = 0; u < 16; ++u) {
      const int i = u * 32 + lane;  // i = l * ksteps + ks: consecutive lanes read consecutive floats
      if (i < total) {
        const int l = i / p.ksteps;
        const int cc = col_of(l);
        if (cc < n) m.v[u] = p.a_scale[static_cast<size_t>(row0 + cc) * p.ksteps + (i - l * p.ksteps)];
      }
    }
  };
  // Weight block scales: those of the CTA's first tiles are read into shared memory by the epilogue warps while the
  // first stages are in flight (a dependent global load issued once the weight stream saturates the memory system
  // takes microseconds, and one per tile was what paced these kernels); tiles past the cache fall back on a
  // register queue loaded two tiles ahead.
  const int ws_per_tile = C::NA * p.ksteps;
  const int ws_ncache = (t_hi - t_lo) < F8_WS_FLOATS / ws_per_tile ? (t_hi - t_lo) : F8_WS_FLOATS / ws_per_tile;
  auto load_ws = [&](int tile, float& w0, float& w1) {
    w0 = w1 = 0.f;
    int e, row0, n, mt;
    if (tile - t_lo < ws_ncache || tile >= t_hi || lane >= p.ksteps || !decode(tile, e, row0, n, mt)) return;
    const float* swb = (e == p.E_local) ? p.s_w_sh : p.s_w + static_cast<size_t>(e) * (p.w_rows / 128) * p.ksteps;
    w0 = swb[static_cast<size_t>(UP ? mt : (MROWS / 128) * mt) * p.ksteps + lane];             // gate / down block row
    if (DUAL) w1 = swb[static_cast<size_t>(UP ? p.I / 128 + mt : 2 * mt + 1) * p.ksteps + lane];  // up rows / next 128 rows
  };
  Meta pre;
  float wsa1 = 0.f, wsb1 = 0.f, wsa2 = 0.f, wsb2 = 0.f;
  if (warp >= 2) {
    fetch(t_lo, pre);
    load_ws(t_lo, wsa1, wsb1);
    load_ws(t_lo + 1, wsa2, wsb2);
  }

  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  if (threadIdx.x == 0) TRACE(3, 0);
#ifdef B200_TRACE
  if (threadIdx.x == 0 && blockIdx.x < 256) { g_cta[blockIdx.x][0] = globaltimer(); g_cta[blockIdx.x][2] = t_hi - t_lo; }
#endif

  if (warp == 0) {
    if (lane == 0) {  // ---------------- TMA producer ----------------
      int stage = 0, issued = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = t_lo; ok && tile < t_hi; ++tile) {
        int e, row0, n, mt;
        if (!decode(tile, e, row0, n, mt)) continue;
        const int nb16 = (n + 15) >> 4;
        const CUtensorMap* mapW = (e == p.E_local) ? &tmWsh : &tmW;
        const int wrow = (e == p.E_local ? 0 : e * p.w_rows) + mt * MROWS;
        const int kfirst = k0_of(tile);
        for (int ks = kfirst; ks < kfirst + kn; ++ks) {
          if (!mbar_wait(&empty[stage], phase ^ 1u, abort_flag, p.status, ST_WAIT_EMPTY)) {
            ok = false;
            break;
          }
          uint8_t* sA = smem + stage * C::STAGE;
          uint8_t* sB = sA + C::NA * F8_TILE;
          // every TMA instruction costs the issuing thread about 100 ns: more than 16 token rows come as ONE box of
          // the mode's largest size (rows past the block belong to the next expert or are zero-filled past the end;
          // the MMA's N ignores them)
          mbar_expect_tx(&full[stage], C::NA * F8_TILE + (WIDE ? F8_TILE : nb16 == 1 ? 2048 : DUAL ? F8_BTILE_MOE : F8_BTILE));
          tma_load_2d(sA, mapW, ks * 128, wrow, &full[stage]);
          if (DUAL) tma_load_2d(sA + F8_TILE, mapW, ks * 128, wrow + (UP ? p.I : 128), &full[stage]);
          if (p.test_starve) {
          } else if (WIDE || nb16 > 1) {   // tmX64 carries the mode's largest box: 128 rows (wide), 32 (expert GEMMs), 64
            tma_load_2d(sB, &tmX64, ks * 128, row0, &full[stage]);
          } else {
            tma_load_2d(sB, &tmX, ks * 128, row0, &full[stage]);
          }
          TRACE(0, issued);
          ++issued;
          if (++stage == C::STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
      if (!ok) {  // abandoned: bounded grace period for the copies in flight
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
    if (lane == 0) {  // ---------------- MMA issuer ----------------
      int stage = 0;
      uint32_t phase = 0, g = 0;  // g counts 128-k blocks over the CTA's whole life
      bool ok = true;
      for (int tile = t_lo; ok && tile < t_hi; ++tile) {
        int e, row0, n, mt;
        if (!decode(tile, e, row0, n, mt)) continue;
        const uint32_t N = static_cast<uint32_t>((n + 15) & ~15);
        const uint32_t idesc = umma_idesc(UMMA_C_F32, UMMA_AB_E4M3, N);
        for (int ks = 0; ks < kn && ok; ++ks, ++g) {
          const uint32_t pb = g % C::NPB, pphase = (g / C::NPB) & 1u;
          if (!mbar_wait(&pempty[pb], pphase ^ 1u, abort_flag, p.status, ST_WAIT_TMEM_EMPTY) ||
              !mbar_wait(&full[stage], phase, abort_flag, p.status, ST_WAIT_FULL)) {
            ok = false;
            break;
          }
          tc_fence_after();
          TRACE(1, g);
          const uint32_t sA = smem_u32(smem + stage * C::STAGE);
          const uint32_t sB = sA + C::NA * F8_TILE;
          const uint32_t d0 = tmem_base + pb * C::PW;
#pragma unroll
          for (int kk = 0; kk < 4; ++kk) {
            const uint64_t db = umma_desc_sw128(sB + kk * 32);
            tc_mma_f8(d0, umma_desc_sw128(sA + kk * 32), db, idesc, kk != 0);
            if (DUAL) tc_mma_f8(d0 + 32, umma_desc_sw128(sA + F8_TILE + kk * 32), db, idesc, kk != 0);
          }
          tc_commit(&empty[stage]);
          tc_commit(&pfull[pb]);
          if (++stage == C::STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
    }
  } else {
    // ---------------- promotion + epilogue: warps 2 and up.  TMEM lane quadrant = warp % 4; the warps of a
    // quadrant share a scheduler and split the tile's columns among them (`half` = which share): two warps with
    // alternate 16-column chunks, or four with 32 consecutive columns each in the wide modes, where the promotion
    // of 128 columns per k block is what paces the kernel and four warps per scheduler hide its latencies.  A
    // thread keeps at most 32 accumulators (16 + 16 in the expert GEMMs) ----------------
    const int q = warp & 3;
    const int half = (warp - 2) >> 2;
    float* m_as = reinterpret_cast<float*>(meta + (warp - 2) * C::META_WARP);  // [ksteps][NL]
    float* m_wt = m_as + (WIDE ? 0 : NL * F8_MAXKG);                           // [32]
    int* m_slot = reinterpret_cast<int*>(m_wt + 32);                           // [32]
    float* m_ws = reinterpret_cast<float*>(m_slot + 32);                       // [2][F8_MAXKG] weight block scales
    const float* __restrict__ a_scale = p.a_scale;
    uint32_t g = 0;
    bool ok = true;
    // local column l of this warp is tile column col_of(l): half * 16 + l (l < 16) in the expert GEMMs,
    // (l / 16) * 32 + half * 16 + l % 16 (l < 32) in the dense modes.
    // Destination row and routing weight of local column `lane` stay in this lane's registers and reach the
    // other lanes by shuffles in the down epilogue (a shared-memory read per stored value there made one
    // dependent round trip per column, 1.7 us per tile).
    bf16* cur_dst = nullptr;
    float cur_wt = 0.f;
    auto stage_block = [&](int row0, int n) {
      const int total = NL * p.ksteps;
#pragma unroll
      for (int u = 0; u < 16; ++u) {
        const int i = u * 32 + lane;
        if (i < total) {
          const int l = i / p.ksteps;
          m_as[(i - l * p.ksteps) * NL + l] = pre.v[u];
        }
      }
      for (int i = 512 + lane; i < total; i += 32) {  // more than 512 scales: the rest is fetched in place
        const int l = i / p.ksteps;
        const int c = col_of(l);
        m_as[(i - l * p.ksteps) * NL + l] = c < n ? a_scale[static_cast<size_t>(row0 + c) * p.ksteps + (i - l * p.ksteps)] : 0.f;
      }
      const int slot = pre.slot < p.total_rows ? pre.slot : -1;
      m_slot[lane] = slot;
      m_wt[lane] = pre.wt;
      if (MODE == MODE_DOWN) {
        bf16* dst = nullptr;
        if (slot >= 0) {
          if (p.ep_world >= 1) {
            const int routed = p.ep_rows * p.ep_world;
            if (slot < routed) {
              const int home = slot / p.ep_rows;
              dst = p.ep_cache[home] + static_cast<size_t>(slot - home * p.ep_rows) * p.H;
            } else {  // shared-expert row of token t: row ep_rows + local t of this rank's own cache
              const int t = slot - routed, home = t / p.ep_tokens;
              if (home == p.ep_rank) dst = p.ep_cache[home] + static_cast<size_t>(p.ep_rows + t - home * p.ep_tokens) * p.H;
            }
          } else {
            dst = p.cache + static_cast<size_t>(slot) * p.H;
          }
        }
        cur_dst = dst;
        cur_wt = pre.wt;
      }
    };
    int staged_blk = -1;
    for (int idx = static_cast<int>(threadIdx.x) - 64; idx < ws_ncache * ws_per_tile; idx += C::THREADS - 64) {
      const int ti = idx / ws_per_tile, rem = idx - ti * ws_per_tile;
      const int which = rem / p.ksteps, ks = rem - which * p.ksteps;
      int e, row0, n, mt;
      float v = 0.f;
      if (decode(t_lo + ti, e, row0, n, mt)) {
        const float* swb = (e == p.E_local) ? p.s_w_sh : p.s_w + static_cast<size_t>(e) * (p.w_rows / 128) * p.ksteps;
        const int srow = UP ? (which ? p.I / 128 + mt : mt) : (MROWS / 128) * mt + which;
        v = swb[static_cast<size_t>(srow) * p.ksteps + ks];
      }
      ws_cache[idx] = v;
    }
    if (WIDE) {   // lane -> row, so the shared-memory writes of a warp fall in consecutive banks
      const int et = static_cast<int>(threadIdx.x) - 64;
      for (int idx = et; idx < tpad * p.ksteps; idx += C::THREADS - 64) {
        const int ks = idx / tpad, row = idx - ks * tpad;
        as_all[idx] = row < p.total_rows ? a_scale[static_cast<size_t>(row) * p.ksteps + ks] : 0.f;
      }
    }
    asm volatile("bar.sync 1, %0;" ::"n"(C::THREADS - 64) : "memory");  // the epilogue warps' fill of ws_cache (and as_all) is complete
    for (int tile = t_lo; ok && tile < t_hi; ++tile) {
      int e, row0, n, mt;
      const bool cached = tile - t_lo < ws_ncache;
      const float ws_a = wsa1, ws_b = wsb1;  // this tile's weight block scales; the queue moves on every tile
      wsa1 = wsa2;
      wsb1 = wsb2;
      load_ws(tile + 2, wsa2, wsb2);  // returns at once for a cached tile
      if (!decode(tile, e, row0, n, mt)) {
        if (lane == 0 && p.status) atomicCAS(p.status, 0, ST_BAD_LIST);
        continue;
      }
      __syncwarp();
      if (warp == 2 && lane == 0) TRACE(5, tile - t_lo);
      const int blk = blk_of(tile);
      if (!WIDE && blk != staged_blk) {  // first tile of a block (dense modes: of a chunk of token rows)
        staged_blk = blk;
        stage_block(row0, n);
        // the next block's metadata is requested now and consumed at that block's first tile
        const int next = LM ? (nblocks > 1 ? tile + 1 : t_hi) : (blk + 1) * p.mtiles;
        fetch(next, pre);
      }
      if (!cached && lane < p.ksteps) {
        m_ws[lane] = ws_a;
        if (DUAL) m_ws[F8_MAXKG + lane] = ws_b;
      }
      __syncwarp();
      const float* __restrict__ wsc_a = cached ? ws_cache + (tile - t_lo) * ws_per_tile : m_ws;
      const float* __restrict__ wsc_b = cached ? wsc_a + p.ksteps : m_ws + F8_MAXKG;
      if (warp == 2 && lane == 0) TRACE(3, 2 + 2 * ((tile - t_lo)));
      float acc_a[NL], acc_b[DUAL ? NL : 1];
#pragma unroll
      for (int c = 0; c < NL; ++c) acc_a[c] = 0.f;
      if (DUAL)
#pragma unroll
        for (int c = 0; c < NL; ++c) acc_b[c] = 0.f;
      const int kfirst = k0_of(tile);
      for (int ks = kfirst; ks < kfirst + kn; ++ks, ++g) {
        const uint32_t pb = g % C::NPB, pphase = (g / C::NPB) & 1u;
        const float wsa = wsc_a[ks], wsb = DUAL ? wsc_b[ks] : 0.f;
        if (!mbar_wait(&pfull[pb], pphase, abort_flag, p.status, ST_WAIT_TMEM_FULL)) {
          ok = false;
          break;
        }
        tc_fence_after();
        if (warp == 2 && lane == 0) TRACE(2, g);
        // chunk h2 (16 columns) of this warp sits at TMEM column tcol(h2) of the partial
        const uint32_t taddr = tmem_base + pb * C::PW + (static_cast<uint32_t>(q * 32) << 16);
        const float* __restrict__ as_w = as_all + ks * tpad + row0 + half * 32;   // wide: scales of this warp's columns
#pragma unroll
        for (int h2 = 0; h2 < NH2; ++h2) {
          const int tcol = WIDE ? half * 32 + h2 * 16 : half * 16 + h2 * 32;
          if (tcol < n) {   // the same for the whole warp
            uint32_t ra[16], rb[16];
            tmem_ld16(taddr + tcol, ra);
            if (DUAL) tmem_ld16(taddr + 32 + tcol, rb);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 16; ++i) {
              const float as = WIDE ? as_w[h2 * 16 + i] : m_as[ks * NL + h2 * 16 + i];
              acc_a[h2 * 16 + i] = __fmaf_rn(__uint_as_float(ra[i]), __fmul_rn(as, wsa), acc_a[h2 * 16 + i]);
              if (DUAL) acc_b[h2 * 16 + i] = __fmaf_rn(__uint_as_float(rb[i]), __fmul_rn(as, wsb), acc_b[h2 * 16 + i]);
            }
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&pempty[pb]);
        if constexpr (DENSE) if (p.partials != nullptr) {
          const int plen = p.ksteps / p.kparts;
          if ((ks + 1) % plen == 0) {   // this part is complete: its sums leave, the accumulators start again from zero
            const int rr = mt * MROWS + q * 32 + lane;
            float* __restrict__ o = p.partials + (static_cast<size_t>(ks / plen) * p.total_rows + row0) * p.w_rows + rr;
#pragma unroll
            for (int l = 0; l < 32; ++l) {
              const int c = col_of(l);
              if (c < n && rr < p.w_rows) st_global_na(o + static_cast<size_t>(c) * p.w_rows, acc_a[l]);
              acc_a[l] = 0.f;
            }
          }
        }
      }
      if (!ok) break;
      if (warp == 2 && lane == 0) TRACE(3, 3 + 2 * ((tile - t_lo)));
      const int r = mt * MROWS + q * 32 + lane;  // down: this lane also holds output feature r + 128
      if constexpr (DENSE) {
        // plain projection: out[token][feature] = bf16(acc)
        if (p.partials != nullptr) {
          // the parts' sums were stored as each part completed
        } else if (r < p.w_rows) {
          int sg = 0;
          while (sg + 1 < p.nseg && r >= p.seg_lo[sg + 1]) ++sg;
          bf16* __restrict__ o = p.seg_out[sg] + (r - p.seg_lo[sg]);
          const size_t ld = static_cast<size_t>(p.seg_ld[sg]);
#pragma unroll
          for (int l = 0; l < 32; ++l) {
            const int c = col_of(l);
            if (c < n) st_global_na(o + static_cast<size_t>(row0 + c) * ld, f2bf(acc_a[l]));
          }
        }
      } else if constexpr (LM) {
        // per token: the largest logit of this warp's 32 vocabulary rows and the lowest row that holds it,
        // as one packed 64-bit key per (tile, quadrant, token); a small kernel takes the max over them.
        // The maximum over the lanes is a transposing butterfly of fmaxf (31 exchanges; NaN never survives
        // against a number, -0 and +0 compare equal), after which lane l holds local column l; the row
        // comes from a ballot of the lanes whose value equals the maximum.
        const bool live = r < p.w_rows;
        auto reduce_cols = [&](const float* acc) {
          float mv[32];
#pragma unroll
          for (int l = 0; l < 32; ++l) {
            mv[l] = live ? acc[l] : __int_as_float(0x7fc00000);
            if (p.lm_logits && live) {
              const int c = col_of(l);
              if (c < n) st_global_na(p.lm_logits + static_cast<size_t>(row0 + c) * p.lm_ld + r, acc[l]);
            }
          }
#pragma unroll
          for (int o = 16; o > 0; o >>= 1) {
            const bool up_half = (lane & o) != 0;
#pragma unroll
            for (int i = 0; i < o; ++i) {
              const float send = up_half ? mv[i] : mv[i + o];
              const float keep = up_half ? mv[i + o] : mv[i];
              mv[i] = fmaxf(keep, __shfl_xor_sync(FULL_MASK, send, o));
            }
          }
          const float best = mv[0];  // column `lane`: NaN only if every live row is NaN (or none is live)
          uint32_t mine = 0u;
#pragma unroll
          for (int l = 0; l < 32; ++l) {
            const float bl = __shfl_sync(FULL_MASK, best, l);
            const uint32_t hit = __ballot_sync(FULL_MASK, live && acc[l] == bl);
            if (lane == l) mine = hit;
          }
          const uint32_t live_mask = __ballot_sync(FULL_MASK, live);
          {
            const int c = col_of(lane);
            if (c < n) {
              unsigned long long key = 0ull;  // no live row
              const int base_id = p.lm_shard_lo + mt * 128 + q * 32;
              if (mine) {
                uint32_t k = __float_as_uint(best + 0.f);
                k = (k & 0x80000000u) ? ~k : (k | 0x80000000u);
                if (k < 2u) k = 2u;
                key = (static_cast<unsigned long long>(k) << 32) |
                      (0xffffffffu - static_cast<uint32_t>(base_id + __ffs(mine) - 1));
              } else if (live_mask) {  // only NaN among the live rows: value part 1, the lowest live row
                key = (1ull << 32) | (0xffffffffu - static_cast<uint32_t>(base_id + __ffs(live_mask) - 1));
              }
              p.lm_keys[(static_cast<size_t>(mt) * 4 + q) * p.total_rows + row0 + c] = key;
            }
          }
        };
        reduce_cols(acc_a);
      } else if constexpr (UP) {
        bf16* __restrict__ hout = p.h_out + static_cast<size_t>(row0) * p.I + r;
#pragma unroll
        for (int l = 0; l < NL; ++l) {
          const int c = col_of(l);
          if (c < n) {
            const float gv = rbf(acc_a[l]), uv = rbf(acc_b[l]);
            const bf16 hv = f2bf(__fmul_rn(__fdiv_rn(gv, 1.f + __expf(-gv)), uv));
            st_global_na(hout + static_cast<size_t>(c) * p.I, hv);
            if (p.dbg_h && m_slot[l] >= 0) st_global_na(p.dbg_h + static_cast<size_t>(m_slot[l]) * p.I + r, hv);
          }
        }
      } else {
#pragma unroll
        for (int l = 0; l < NL; ++l) {
          const int c = col_of(l);
          if (c < n) {  // the same for every lane of the warp
            bf16* dst = reinterpret_cast<bf16*>(__shfl_sync(FULL_MASK, reinterpret_cast<unsigned long long>(cur_dst), l));
            const float wt = __shfl_sync(FULL_MASK, cur_wt, l);
            if (dst != nullptr) {
              st_global_na(dst + r, f2bf(__fmul_rn(acc_a[l], wt)));
              st_global_na(dst + r + 128, f2bf(__fmul_rn(acc_b[l], wt)));
            }
          }
        }
      }
      if (warp == 2 && lane == 0) TRACE(4, tile - t_lo);
    }
  }
  if (warp == 2 && lane == 0) TRACE(3, 1);
#ifdef B200_TRACE
  if (warp == 2 && lane == 0 && blockIdx.x < 256) g_cta[blockIdx.x][1] = globaltimer();
#endif
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, C::TMEM);
  }
}

#ifdef B200_TRACE
extern "C" int b200_trace_read(unsigned long long* host) {
  return static_cast<int>(cudaMemcpyFromSymbol(host, g_trace, sizeof(g_trace)));
}
extern "C" int b200_trace_read_cta(unsigned long long* host) {
  return static_cast<int>(cudaMemcpyFromSymbol(host, g_cta, sizeof(g_cta)));
}
#endif

// x bf16 [T, H] -> e4m3 rows [T, H] + scales [T, H/128] in token order (no permutation)
void b200_quant_rows_f8_launch(const void* x, int T, int H, uint8_t* xq, float* xs, cudaStream_t st) {
  quant_permute_f8_kernel<<<T, 256, 0, st>>>(static_cast<const bf16*>(x), T, H, 0, nullptr, 0, T, xq, xs, F8Partition{});
}

struct F8Layout {
  size_t xq, xs, h, hq, hs, part, total;
};
static F8Layout f8_layout(int T, int H, int I, int K) {
  const size_t rows = static_cast<size_t>(T) * (K + 1);
  auto up = [](size_t v) { return (v + 1023) & ~size_t(1023); };
  F8Layout l;
  size_t o = 0;
  l.xq = o; o = up(o + rows * H);
  l.xs = o; o = up(o + rows * (H / 128) * 4);
  l.h = o;  o = up(o + rows * I * 2);
  l.hq = o; o = up(o + rows * I);
  l.hs = o; o = up(o + rows * (I / 128) * 4);
  l.part = o; o = up(o + 2 * F8_PART_INTS * 4);
  l.total = o;
  return l;
}

}  // namespace b200

using namespace b200;

extern "C" size_t b200_moe_fp8_workspace_bytes(int T, int H, int I, int K) {
  if (T <= 0 || H <= 0 || I <= 0 || K <= 0) return 0;
  return f8_layout(T, H, I, K).total;
}

static int moe_fp8_impl(const void* x, int T, int H, int I, int K, int E_local, const b200_moe_weights* w,
                        const b200_moe_lists* lists, void* cache, void* ws, size_t ws_bytes, void* dbg_h, int stages,
                        int32_t* status, void* stream, void* const* peer_cache, int ep_world, int ep_rank,
                        int ep_tokens_per_rank) {
  if (!x || !w || !lists || !cache || !ws || !w->w13 || !w->s13 || !w->w2 || !w->s2)
    return fail(B200_E_ARG, "b200_moe_fp8: null pointer");
  if (T <= 0 || K <= 0 || K > 32 || E_local <= 0 || H % 256 || I % 128 || H <= 0 || I <= 0 || H / 128 > F8_MAXKG ||
      I / 128 > F8_MAXKG)
    return fail(B200_E_ARG, "b200_moe_fp8: need H a multiple of 256, I of 128, both <= 4096, 1 <= K <= 32 (T=%d H=%d I=%d K=%d)",
                T, H, I, K);
  const F8Layout l = f8_layout(T, H, I, K);
  if (ws_bytes < l.total) return fail(B200_E_WS, "b200_moe_fp8: workspace %zu < %zu bytes", ws_bytes, l.total);
  if (reinterpret_cast<uintptr_t>(ws) & 1023) return fail(B200_E_ALIGN, "b200_moe_fp8: workspace must be 1024-byte aligned");
  if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(cache)) & 15)
    return fail(B200_E_ALIGN, "b200_moe_fp8: x and cache must be 16-byte aligned");
  const bool shared = w->sh13 != nullptr;
  if (shared && (!w->shs13 || !w->sh2 || !w->shs2)) return fail(B200_E_ARG, "b200_moe_fp8: incomplete shared expert");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  uint8_t* base = static_cast<uint8_t*>(ws);
  uint8_t* xq = base + l.xq;
  float* xs = reinterpret_cast<float*>(base + l.xs);
  bf16* h = reinterpret_cast<bf16*>(base + l.h);
  uint8_t* hq = base + l.hq;
  float* hs = reinterpret_cast<float*>(base + l.hs);
  const int rows = T * (K + 1);
  MoeLists L{lists->counts,     lists->offsets,  lists->row_of_pair, lists->slot_of_row, lists->wt_of_row,
             lists->blk_expert, lists->blk_row0, lists->blk_rows,    lists->nblocks};
  CUtensorMap tmW13, tmSh13, tmXq, tmXq64, tmW2, tmSh2, tmHq, tmHq64;
  int rc;
  if ((rc = make_tmap_bytes_2d(&tmW13, w->w13, static_cast<uint64_t>(E_local) * 2 * I, H, 128, "w13"))) return rc;
  if ((rc = make_tmap_bytes_2d(&tmSh13, shared ? w->sh13 : w->w13, 2 * I, H, 128, "sh13"))) return rc;
  if ((rc = make_tmap_bytes_2d(&tmXq, xq, rows, H, 16, "xq"))) return rc;
  if ((rc = make_tmap_bytes_2d(&tmXq64, xq, rows, H, 32, "xq"))) return rc;   // the largest block: 32 rows
  if ((rc = make_tmap_bytes_2d(&tmW2, w->w2, static_cast<uint64_t>(E_local) * H, I, 128, "w2"))) return rc;
  if ((rc = make_tmap_bytes_2d(&tmSh2, shared ? w->sh2 : w->w2, H, I, 128, "sh2"))) return rc;
  if ((rc = make_tmap_bytes_2d(&tmHq, hq, rows, I, 16, "hq"))) return rc;
  if ((rc = make_tmap_bytes_2d(&tmHq64, hq, rows, I, 32, "hq"))) return rc;
  static DeviceOnce once;
  once.run([] {
    cudaFuncSetAttribute(moe_gemm_f8_kernel<MODE_UP>, cudaFuncAttributeMaxDynamicSharedMemorySize, F8Cfg<MODE_UP>::SMEM);
    cudaFuncSetAttribute(moe_gemm_f8_kernel<MODE_DOWN>, cudaFuncAttributeMaxDynamicSharedMemorySize, F8Cfg<MODE_DOWN>::SMEM);
  });
  if ((stages & 15) == 0) stages |= 15;
  // tokens that get a shared-expert row: all of them, or this rank's own under expert parallelism
  int shared_lo = 0, shared_n = shared ? T : 0;
  if (ep_world >= 1 && shared) {
    shared_lo = ep_rank * ep_tokens_per_rank;
    shared_n = ep_tokens_per_rank;
  }
  const int grid = sm_count();
  // the quantiser's launch carries one extra CTA that cuts the tile sequences of the two GEMMs over their CTAs; a call
  // without the quantise stage leaves that to every GEMM CTA itself
  int32_t* part = reinterpret_cast<int32_t*>(base + l.part);
  const bool with_part = (stages & B200_MOE_STAGE_QUANT) && grid + 1 <= F8_PART_INTS;
  if (stages & B200_MOE_STAGE_QUANT) {
    F8Partition q{};
    q.blk_rows = L.blk_rows;
    q.nblocks = L.nblocks;
    q.grid = grid;
    q.mtiles[0] = I / 128;
    q.cost_base[0] = 7;
    q.mtiles[1] = H / 256;
    q.cost_base[1] = 5;
    q.table[0] = part;
    q.table[1] = part + F8_PART_INTS;
    quant_permute_f8_kernel<<<T + (with_part ? 1 : 0), 256, 0, st>>>(static_cast<const bf16*>(x), T, H, K, L.row_of_pair,
                                                                    shared_lo, shared_n, xq, xs, q);
  }
  F8Args a{};
  a.L = L;
  a.E_local = E_local;
  a.I = I;
  a.H = H;
  a.total_rows = rows;
  a.status = status;
  a.test_starve = (stages & B200_MOE_TEST_STARVE) ? 1 : 0;
  a.mtiles = I / 128;
  a.ksteps = H / 128;
  a.w_rows = 2 * I;
  a.cost_base = 7;   // a tile costs 7 + 16-row units of its block (a sweep of 1..30 moved the kernel by less than 2 %)
  a.part = with_part ? part : nullptr;
  a.s_w = w->s13;
  a.s_w_sh = w->shs13;
  a.a_scale = xs;
  a.h_out = h;
  a.dbg_h = static_cast<bf16*>(dbg_h);
  if (stages & B200_MOE_STAGE_UP)
    moe_gemm_f8_kernel<MODE_UP><<<grid, F8_THREADS, F8Cfg<MODE_UP>::SMEM, st>>>(tmW13, tmSh13, tmXq, tmXq64, a);
  if (stages & B200_MOE_STAGE_HQUANT)
    quant_rows_f8_kernel<<<(rows + 7) / 8, 256, 0, st>>>(h, rows, I, L.slot_of_row, hq, hs);
  a.mtiles = H / 256;  // two consecutive 128-row tiles of W2 per GEMM tile
  a.ksteps = I / 128;
  a.w_rows = H;
  a.cost_base = 5;
  a.part = with_part ? part + F8_PART_INTS : nullptr;
  a.s_w = w->s2;
  a.s_w_sh = w->shs2;
  a.a_scale = hs;
  a.h_out = nullptr;
  a.cache = static_cast<bf16*>(cache);
  a.dbg_h = nullptr;
  a.ep_world = ep_world;
  a.ep_rank = ep_rank;
  a.ep_tokens = ep_tokens_per_rank;
  a.ep_rows = ep_tokens_per_rank * K;
  for (int r = 0; r < 8; ++r) a.ep_cache[r] = (peer_cache && r < ep_world) ? static_cast<bf16*>(peer_cache[r]) : nullptr;
  if (stages & B200_MOE_STAGE_DOWN)
    moe_gemm_f8_kernel<MODE_DOWN><<<grid, F8_THREADS, F8Cfg<MODE_DOWN>::SMEM, st>>>(tmW2, tmSh2, tmHq, tmHq64, a);
  return launch_status("b200_moe_fp8");
}

extern "C" int b200_moe_fp8(const void* x, int T, int H, int I, int K, int E_local, const b200_moe_weights* w,
                            const b200_moe_lists* lists, void* cache, void* ws, size_t ws_bytes, void* dbg_h,
                            int stages, int32_t* status, void* stream) {
  return moe_fp8_impl(x, T, H, I, K, E_local, w, lists, cache, ws, ws_bytes, dbg_h, stages, status, stream, nullptr, 0, 0,
                      0);
}

extern "C" int b200_moe_fp8_ep(const void* x, int T, int H, int I, int K, int E_local, const b200_moe_weights* w,
                               const b200_moe_lists* lists, void* const* peer_cache_host, int ep_world, int ep_rank,
                               int ep_tokens_per_rank, void* ws, size_t ws_bytes, int32_t* status, void* stream) {
  if (!peer_cache_host || ep_world < 1 || ep_world > 8 || ep_rank < 0 || ep_rank >= ep_world || ep_tokens_per_rank <= 0 ||
      T != ep_world * ep_tokens_per_rank)
    return fail(B200_E_ARG, "b200_moe_fp8_ep: need 1 <= ep_world <= 8, 0 <= ep_rank < ep_world and T == ep_world * "
                "ep_tokens_per_rank (T=%d)", T);
  for (int r = 0; r < ep_world; ++r)
    if (!peer_cache_host[r] || (reinterpret_cast<uintptr_t>(peer_cache_host[r]) & 15))
      return fail(B200_E_ARG, "b200_moe_fp8_ep: peer cache %d is null or not 16-byte aligned", r);
  return moe_fp8_impl(x, T, H, I, K, E_local, w, lists, peer_cache_host[ep_rank], ws, ws_bytes, nullptr, 0, status, stream,
                      peer_cache_host, ep_world, ep_rank, ep_tokens_per_rank);
}

// ---- LM head shard with fused argmax ------------------------------------------------------------------
namespace b200 {
__global__ void __launch_bounds__(256) lmhead_finish_kernel(const unsigned long long* __restrict__ keys, int parts, int T,
                                                            float* __restrict__ max_out, int32_t* __restrict__ idx_out) {
  // one CTA per token: max over the (tile, warp) partial keys
  __shared__ unsigned long long red[8];
  const int t = blockIdx.x, tid = threadIdx.x, lane = tid & 31;
  pdl_wait();
  pdl_launch();
  unsigned long long k = 0ull;
  for (int i = tid; i < parts; i += 256) {
    const unsigned long long v = keys[static_cast<size_t>(i) * T + t];
    k = v > k ? v : k;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const unsigned long long v = __shfl_xor_sync(FULL_MASK, k, o);
    k = v > k ? v : k;
  }
  if (lane == 0) red[tid >> 5] = k;
  __syncthreads();
  if (tid != 0) return;
  for (int w = 1; w < 8; ++w) k = red[w] > k ? red[w] : k;
  const uint32_t m = static_cast<uint32_t>(k >> 32);
  float v;
  if (m <= 1u)
    v = __int_as_float(0x7fc00000);  // no finite candidate in this shard
  else
    v = __uint_as_float((m & 0x80000000u) ? (m & 0x7fffffffu) : ~m);
  max_out[t] = v;
  idx_out[t] = m == 0u ? -1 : static_cast<int32_t>(0xffffffffu - static_cast<uint32_t>(k & 0xffffffffull));
}

// tokens[t] = id of the largest value over the S shards; ties to the lower id; NaN never wins
__global__ void argmax_merge_kernel(const float* __restrict__ maxes, const int32_t* __restrict__ idxs, int S, int T,
                                    int32_t* __restrict__ tokens) {
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= T) return;
  float best = 0.f;
  int id = -1;
  for (int s = 0; s < S; ++s) {
    const float v = maxes[static_cast<size_t>(s) * T + t];
    const int i = idxs[static_cast<size_t>(s) * T + t];
    if (i < 0 || v != v) continue;
    if (id < 0 || v > best || (v == best && i < id)) {
      best = v;
      id = i;
    }
  }
  if (id < 0)
    for (int s = 0; s < S; ++s) {
      const int i = idxs[static_cast<size_t>(s) * T + t];
      if (i >= 0 && (id < 0 || i < id)) id = i;
    }
  tokens[t] = id;
}

struct LmLayout {
  size_t xq, xs, keys, total;
};
// The dense modes take 128-row chunks when there are more than 64 rows and the activation scales of all rows fit
// the kernel's shared-memory table; the per-element arithmetic is the same either way.
static bool dense_wide(int T, int K) { return T > 64 && ((T + 127) / 128) * 128 * (K / 128) <= F8_AS_FLOATS; }
static int dense_chunks(int T, int K) { return dense_wide(T, K) ? (T + 127) / 128 : (T + 63) / 64; }
template <int NARROW, int WIDEM>
static void launch_dense(bool wide, int grid, const CUtensorMap& tmW, const CUtensorMap& tmX, const CUtensorMap& tmXbox,
                         const F8Args& a, cudaStream_t st) {
  static DeviceOnce once;
  once.run([] {
    cudaFuncSetAttribute(moe_gemm_f8_kernel<NARROW>, cudaFuncAttributeMaxDynamicSharedMemorySize, F8Cfg<NARROW>::SMEM);
    cudaFuncSetAttribute(moe_gemm_f8_kernel<WIDEM>, cudaFuncAttributeMaxDynamicSharedMemorySize, F8Cfg<WIDEM>::SMEM);
  });
  if (wide)
    moe_gemm_f8_kernel<WIDEM><<<grid, F8Cfg<WIDEM>::THREADS, F8Cfg<WIDEM>::SMEM, st>>>(tmW, tmW, tmX, tmXbox, a);
  else
    moe_gemm_f8_kernel<NARROW><<<grid, F8_THREADS, F8Cfg<NARROW>::SMEM, st>>>(tmW, tmW, tmX, tmXbox, a);
}
static LmLayout lm_layout(int T, int H, int V_shard) {
  auto up = [](size_t v) { return (v + 1023) & ~size_t(1023); };
  LmLayout l;
  size_t o = 0;
  l.xq = o; o = up(o + static_cast<size_t>(T < 64 ? 64 : T) * H);  // at least 64 rows
  l.xs = o; o = up(o + static_cast<size_t>(T) * (H / 128) * 4);
  l.keys = o; o = up(o + static_cast<size_t>((V_shard + 127) / 128) * 4 * T * 8);
  l.total = o;
  return l;
}
}  // namespace b200

extern "C" size_t b200_lmhead_workspace_bytes(int T, int H, int V_shard) {
  if (T <= 0 || H <= 0 || V_shard <= 0) return 0;
  return lm_layout(T, H, V_shard).total;
}

extern "C" int b200_lmhead_argmax(const void* x, int T, int H, const void* w, const float* w_s, int V_shard,
                                  int shard_lo, float* max_out, int32_t* idx_out, float* logits_out, void* ws,
                                  size_t ws_bytes, int32_t* status, void* stream) {
  if (!x || !w || !w_s || !max_out || !idx_out || !ws) return fail(B200_E_ARG, "b200_lmhead_argmax: null pointer");
  if (T <= 0 || H <= 0 || H % 128 || H / 128 > F8_MAXKG || V_shard <= 0 || shard_lo < 0)
    return fail(B200_E_ARG, "b200_lmhead_argmax: need T >= 1, H %% 128 == 0, H <= 4096 (T=%d H=%d V=%d)", T, H, V_shard);
  const LmLayout l = lm_layout(T, H, V_shard);
  if (ws_bytes < l.total) return fail(B200_E_WS, "b200_lmhead_argmax: workspace %zu < %zu bytes", ws_bytes, l.total);
  if (reinterpret_cast<uintptr_t>(ws) & 1023) return fail(B200_E_ALIGN, "b200_lmhead_argmax: workspace must be 1024-byte aligned");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  uint8_t* base = static_cast<uint8_t*>(ws);
  uint8_t* xq = base + l.xq;
  float* xs = reinterpret_cast<float*>(base + l.xs);
  unsigned long long* keys = reinterpret_cast<unsigned long long*>(base + l.keys);
  CUtensorMap tmW, tmX, tmX64;
  int rc;
  if ((rc = make_tmap_bytes_2d(&tmW, w, static_cast<uint64_t>(V_shard), H, 128, "lm_head weight"))) return rc;
  if ((rc = make_tmap_bytes_2d(&tmX, xq, T, H, 16, "lm_head activations"))) return rc;
  const bool wide = dense_wide(T, H);
  if ((rc = make_tmap_bytes_2d(&tmX64, xq, T, H, wide ? 128 : 64, "lm_head activations"))) return rc;
  // K = 0 routed picks: the "shared expert" row of token t is row t
  quant_permute_f8_kernel<<<T, 256, 0, st>>>(static_cast<const bf16*>(x), T, H, 0, nullptr, 0, T, xq, xs, F8Partition{});
  F8Args a{};
  a.E_local = 1;
  a.mtiles = (V_shard + 127) / 128;
  a.ksteps = H / 128;
  a.w_rows = V_shard;
  a.I = 0;
  a.H = H;
  a.total_rows = T;   // more than 64 rows: 64- or 128-row chunks, every weight tile against each chunk in turn
  a.s_w = w_s;
  a.s_w_sh = w_s;
  a.a_scale = xs;
  a.status = status;
  a.lm_keys = keys;
  a.lm_logits = logits_out;
  a.lm_ld = V_shard;
  a.lm_shard_lo = shard_lo;
  const int ntiles = a.mtiles * dense_chunks(T, H);
  const int grid = ntiles < sm_count() ? ntiles : sm_count();
  launch_dense<MODE_LM, MODE_LM_W>(wide, grid, tmW, tmX, tmX64, a, st);
  launch_k(lmhead_finish_kernel, dim3(T), dim3(256), 0, st, static_cast<const unsigned long long*>(keys), a.mtiles * 4, T,
           max_out, idx_out);
  return launch_status("b200_lmhead_argmax");
}

extern "C" int b200_argmax_merge(const float* maxes, const int32_t* idxs, int S, int T, int32_t* tokens, void* stream) {
  if (!maxes || !idxs || !tokens) return fail(B200_E_ARG, "b200_argmax_merge: null pointer");
  if (S <= 0 || T < 0) return fail(B200_E_ARG, "b200_argmax_merge: bad shape (S=%d T=%d)", S, T);
  if (T == 0) return 0;
  argmax_merge_kernel<<<(T + 127) / 128, 128, 0, static_cast<cudaStream_t>(stream)>>>(maxes, idxs, S, T, tokens);
  return launch_status("b200_argmax_merge");
}

// ---- dense decode-width projection (fp8 block-scaled weight, <= 64 rows) and the add + norm after it ----
namespace b200 {
// r = bf16(proj + residual) (the projection is already rounded to bf16; the add is fp32), written back to
// `residual`; y = bf16(r * rsqrt(mean r^2 + eps) * (1 + w)).  One CTA per row.
__global__ void __launch_bounds__(256) add_rmsnorm_kernel(const bf16* __restrict__ proj, bf16* __restrict__ residual,
                                                          const bf16* __restrict__ w, float eps, int H,
                                                          bf16* __restrict__ out) {
  __shared__ float red[8];
  const int t = blockIdx.x, tid = threadIdx.x;
  float ss = 0.f;
  for (int c = tid * 8; c < H; c += 2048) {
    const uint4 a = *reinterpret_cast<const uint4*>(proj + static_cast<size_t>(t) * H + c);
    const uint4 b = *reinterpret_cast<const uint4*>(residual + static_cast<size_t>(t) * H + c);
    float r[8] = {rbf(bf_lo(a.x) + bf_lo(b.x)), rbf(bf_hi(a.x) + bf_hi(b.x)), rbf(bf_lo(a.y) + bf_lo(b.y)),
                  rbf(bf_hi(a.y) + bf_hi(b.y)), rbf(bf_lo(a.z) + bf_lo(b.z)), rbf(bf_hi(a.z) + bf_hi(b.z)),
                  rbf(bf_lo(a.w) + bf_lo(b.w)), rbf(bf_hi(a.w) + bf_hi(b.w))};
#pragma unroll
    for (int i = 0; i < 8; ++i) ss = fmaf(r[i], r[i], ss);
    *reinterpret_cast<uint4*>(residual + static_cast<size_t>(t) * H + c) =
        make_uint4(pack_bf2(r[0], r[1]), pack_bf2(r[2], r[3]), pack_bf2(r[4], r[5]), pack_bf2(r[6], r[7]));
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(FULL_MASK, ss, o);
  if ((tid & 31) == 0) red[tid >> 5] = ss;
  __syncthreads();
  float tot = 0.f;
  for (int i = 0; i < 8; ++i) tot += red[i];
  const float rstd = rsqrtf(tot / H + eps);
  for (int c = tid * 8; c < H; c += 2048) {  // each thread re-reads the rows it wrote itself
    const uint4 b = *reinterpret_cast<const uint4*>(residual + static_cast<size_t>(t) * H + c);
    const uint4 g = *reinterpret_cast<const uint4*>(w + c);
    const float r[8] = {bf_lo(b.x), bf_hi(b.x), bf_lo(b.y), bf_hi(b.y), bf_lo(b.z), bf_hi(b.z), bf_lo(b.w), bf_hi(b.w)};
    const float gw[8] = {bf_lo(g.x), bf_hi(g.x), bf_lo(g.y), bf_hi(g.y), bf_lo(g.z), bf_hi(g.z), bf_lo(g.w), bf_hi(g.w)};
    float y[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) y[i] = r[i] * rstd * (1.f + gw[i]);
    *reinterpret_cast<uint4*>(out + static_cast<size_t>(t) * H + c) =
        make_uint4(pack_bf2(y[0], y[1]), pack_bf2(y[2], y[3]), pack_bf2(y[4], y[5]), pack_bf2(y[6], y[7]));
  }
}
}  // namespace b200

extern "C" size_t b200_dense_fp8_workspace_bytes(int T, int H) {
  if (T <= 0 || H <= 0) return 0;
  auto up = [](size_t v) { return (v + 1023) & ~size_t(1023); };
  return up(static_cast<size_t>(T < 64 ? 64 : T) * H) + up(static_cast<size_t>(T) * (H / 128) * 4);
}

// `x` bf16 rows quantised here into `ws`, or (x == nullptr) rows that arrive as e4m3 `xq_in` + scales `xs_in`
static int dense_split_impl(const void* x, const void* xq_in, const float* xs_in, int T, int H, const void* w,
                            const float* w_s, int N, int nseg, const int* seg_cols_host, void* const* seg_out_host,
                            const int* seg_ld_host, void* ws, size_t ws_bytes, int32_t* status, void* stream) {
  const bool pre = x == nullptr;
  if ((!pre && !ws) || (pre && (!xq_in || !xs_in)) || !w || !w_s || !seg_cols_host || !seg_out_host || !seg_ld_host)
    return fail(B200_E_ARG, "b200_dense_fp8: null pointer");
  if (T <= 0 || H <= 0 || H % 128 || H / 128 > F8_MAXKG || N <= 0 || nseg < 1 || nseg > 4)
    return fail(B200_E_ARG, "b200_dense_fp8: need T >= 1, H %% 128 == 0, H <= 4096, 1 <= segments <= 4 (T=%d H=%d N=%d)", T,
                H, N);
  int lo = 0;
  for (int i = 0; i < nseg; ++i) {
    if (seg_cols_host[i] <= 0 || (i + 1 < nseg && seg_cols_host[i] % 32) || !seg_out_host[i] ||
        seg_ld_host[i] < seg_cols_host[i])
      return fail(B200_E_ARG, "b200_dense_fp8: segment %d: width must be positive (a multiple of 32 except the last), its "
                  "row pitch at least the width, its output non-null", i);
    lo += seg_cols_host[i];
  }
  if (lo != N) return fail(B200_E_ARG, "b200_dense_fp8: segment widths add up to %d, N = %d", lo, N);
  if (!pre && ws_bytes < b200_dense_fp8_workspace_bytes(T, H))
    return fail(B200_E_WS, "b200_dense_fp8: workspace %zu < %zu bytes", ws_bytes, b200_dense_fp8_workspace_bytes(T, H));
  if (!pre && (reinterpret_cast<uintptr_t>(ws) & 1023))
    return fail(B200_E_ALIGN, "b200_dense_fp8: workspace must be 1024-byte aligned");
  if (pre && (reinterpret_cast<uintptr_t>(xq_in) & 15))
    return fail(B200_E_ALIGN, "b200_dense_fp8_split_q: the e4m3 rows must be 16-byte aligned");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const uint8_t* xq = pre ? static_cast<const uint8_t*>(xq_in) : static_cast<uint8_t*>(ws);
  const float* xs = pre ? xs_in
                        : reinterpret_cast<float*>(static_cast<uint8_t*>(ws) +
                                                   ((static_cast<size_t>(T < 64 ? 64 : T) * H + 1023) & ~size_t(1023)));
  CUtensorMap tmW, tmX, tmX64;
  int rc;
  if ((rc = make_tmap_bytes_2d(&tmW, w, static_cast<uint64_t>(N), H, 128, "dense weight"))) return rc;
  if ((rc = make_tmap_bytes_2d(&tmX, xq, T, H, 16, "dense activations"))) return rc;
  const bool wide = dense_wide(T, H);
  if ((rc = make_tmap_bytes_2d(&tmX64, xq, T, H, wide ? 128 : 64, "dense activations"))) return rc;
  if (!pre)
    quant_permute_f8_kernel<<<T, 256, 0, st>>>(static_cast<const bf16*>(x), T, H, 0, nullptr, 0, T, const_cast<uint8_t*>(xq),
                                               const_cast<float*>(xs), F8Partition{});
  F8Args a{};
  a.E_local = 1;
  a.mtiles = (N + 127) / 128;
  a.ksteps = H / 128;
  a.w_rows = N;
  a.H = H;
  a.total_rows = T;   // more than 64 rows: 64- or 128-row chunks, every weight tile against each chunk in turn
  a.s_w = w_s;
  a.s_w_sh = w_s;
  a.a_scale = xs;
  a.status = status;
  a.ksplit = 1;
  a.kparts = 1;
  a.nseg = nseg;
  int c0 = 0;
  for (int i = 0; i < nseg; ++i) {
    a.seg_lo[i] = c0;
    a.seg_ld[i] = seg_ld_host[i];
    a.seg_out[i] = static_cast<bf16*>(seg_out_host[i]);
    c0 += seg_cols_host[i];
  }
  a.seg_lo[nseg] = c0;
  const int ntiles = a.mtiles * dense_chunks(T, H);
  const int grid = ntiles < sm_count() ? ntiles : sm_count();
  launch_dense<MODE_DENSE, MODE_DENSE_W>(wide, grid, tmW, tmX, tmX64, a, st);
  return launch_status("b200_dense_fp8");
}

extern "C" int b200_dense_fp8_split(const void* x, int T, int H, const void* w, const float* w_s, int N, int nseg,
                                    const int* seg_cols_host, void* const* seg_out_host, const int* seg_ld_host, void* ws,
                                    size_t ws_bytes, int32_t* status, void* stream) {
  if (!x) return fail(B200_E_ARG, "b200_dense_fp8: null pointer");
  return dense_split_impl(x, nullptr, nullptr, T, H, w, w_s, N, nseg, seg_cols_host, seg_out_host, seg_ld_host, ws, ws_bytes,
                          status, stream);
}

extern "C" int b200_dense_fp8_split_q(const void* xq, const float* xs, int T, int H, const void* w, const float* w_s, int N,
                                      int nseg, const int* seg_cols_host, void* const* seg_out_host, const int* seg_ld_host,
                                      int32_t* status, void* stream) {
  return dense_split_impl(nullptr, xq, xs, T, H, w, w_s, N, nseg, seg_cols_host, seg_out_host, seg_ld_host, nullptr, 0, status,
                          stream);
}

extern "C" int b200_dense_fp8(const void* x, int T, int H, const void* w, const float* w_s, int N, void* out, void* ws,
                              size_t ws_bytes, int32_t* status, void* stream) {
  if (!out) return fail(B200_E_ARG, "b200_dense_fp8: null pointer");
  void* outs[1] = {out};
  return b200_dense_fp8_split(x, T, H, w, w_s, N, 1, &N, outs, &N, ws, ws_bytes, status, stream);
}

namespace b200 {
// The add + norm behind a split-K projection: proj = bf16(sum of the S partial rows, in split order), then as
// add_rmsnorm_kernel.  One CTA per row.
__global__ void __launch_bounds__(256) add_rmsnorm_partials_kernel(const float* __restrict__ partials, int S, int T,
                                                                   bf16* __restrict__ residual, const bf16* __restrict__ w,
                                                                   float eps, int H, bf16* __restrict__ out,
                                                                   bf16* __restrict__ proj_out) {
  __shared__ float red[8];
  const int t = blockIdx.x, tid = threadIdx.x;
  float ss = 0.f;
  for (int c = tid * 8; c < H; c += 2048) {
    float p[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int s = 0; s < S; ++s) {
      const float4* src = reinterpret_cast<const float4*>(partials + (static_cast<size_t>(s) * T + t) * H + c);
      const float4 a = src[0], b = src[1];
      p[0] += a.x; p[1] += a.y; p[2] += a.z; p[3] += a.w;
      p[4] += b.x; p[5] += b.y; p[6] += b.z; p[7] += b.w;
    }
    const uint4 rb = *reinterpret_cast<const uint4*>(residual + static_cast<size_t>(t) * H + c);
    const float rv[8] = {bf_lo(rb.x), bf_hi(rb.x), bf_lo(rb.y), bf_hi(rb.y), bf_lo(rb.z), bf_hi(rb.z), bf_lo(rb.w), bf_hi(rb.w)};
    float r[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      p[i] = rbf(p[i]);                 // the projection is rounded to bf16 before the fp32 residual add (proj.py:75-77)
      r[i] = rbf(p[i] + rv[i]);
      ss = fmaf(r[i], r[i], ss);
    }
    if (proj_out)
      *reinterpret_cast<uint4*>(proj_out + static_cast<size_t>(t) * H + c) =
          make_uint4(pack_bf2(p[0], p[1]), pack_bf2(p[2], p[3]), pack_bf2(p[4], p[5]), pack_bf2(p[6], p[7]));
    *reinterpret_cast<uint4*>(residual + static_cast<size_t>(t) * H + c) =
        make_uint4(pack_bf2(r[0], r[1]), pack_bf2(r[2], r[3]), pack_bf2(r[4], r[5]), pack_bf2(r[6], r[7]));
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(FULL_MASK, ss, o);
  if ((tid & 31) == 0) red[tid >> 5] = ss;
  __syncthreads();
  float tot = 0.f;
  for (int i = 0; i < 8; ++i) tot += red[i];
  const float rstd = rsqrtf(tot / H + eps);
  for (int c = tid * 8; c < H; c += 2048) {  // each thread re-reads the rows it wrote itself
    const uint4 b = *reinterpret_cast<const uint4*>(residual + static_cast<size_t>(t) * H + c);
    const uint4 g = *reinterpret_cast<const uint4*>(w + c);
    const float r[8] = {bf_lo(b.x), bf_hi(b.x), bf_lo(b.y), bf_hi(b.y), bf_lo(b.z), bf_hi(b.z), bf_lo(b.w), bf_hi(b.w)};
    const float gw[8] = {bf_lo(g.x), bf_hi(g.x), bf_lo(g.y), bf_hi(g.y), bf_lo(g.z), bf_hi(g.z), bf_lo(g.w), bf_hi(g.w)};
    float y[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) y[i] = r[i] * rstd * (1.f + gw[i]);
    *reinterpret_cast<uint4*>(out + static_cast<size_t>(t) * H + c) =
        make_uint4(pack_bf2(y[0], y[1]), pack_bf2(y[2], y[3]), pack_bf2(y[4], y[5]), pack_bf2(y[6], y[7]));
  }
}

// K parts of the projection in front of an add + norm: as many as would let weight tiles x parts fill the GPU at the
// smallest batch.  The part count fixes the arithmetic (a row's sum does not depend on the batch it is in); over how
// many CTAs the parts of one (weight tile, row chunk) are spread is a scheduling choice that shrinks as the rows grow.
static int proj_kparts(int N, int K) {
  const int mtiles = (N + 127) / 128, ksteps = K / 128;
  int s = 1;
  while (s * 2 <= ksteps && ksteps % (s * 2) == 0 && mtiles * s * 2 <= 148) s *= 2;
  return s;
}
static int proj_ksplit(int N, int K, int T) {
  const int units = ((N + 127) / 128) * dense_chunks(T, K);
  int s = proj_kparts(N, K);
  while (s > 1 && units * s > sm_count()) s >>= 1;
  return s;
}
}  // namespace b200

extern "C" size_t b200_dense_fp8_add_rmsnorm_workspace_bytes(int T, int K, int N) {
  if (T <= 0 || K <= 0 || N <= 0 || K % 128) return 0;
  auto up = [](size_t v) { return (v + 1023) & ~size_t(1023); };
  return b200_dense_fp8_workspace_bytes(T, K) + up(static_cast<size_t>(proj_kparts(N, K)) * T * N * 4);
}

extern "C" int b200_dense_fp8_add_rmsnorm(const void* x, int T, int K, const void* w, const float* w_s, int N, void* residual,
                                          const void* norm_w, float eps, void* out, void* proj_out, void* ws,
                                          size_t ws_bytes, int32_t* status, void* stream) {
  if (!x || !w || !w_s || !residual || !norm_w || !out || !ws) return fail(B200_E_ARG, "b200_dense_fp8_add_rmsnorm: null pointer");
  if (T <= 0 || K <= 0 || K % 128 || K / 128 > F8_MAXKG || N <= 0 || N % 8)
    return fail(B200_E_ARG, "b200_dense_fp8_add_rmsnorm: need T >= 1, K %% 128 == 0, K <= 4096, N %% 8 == 0 (T=%d K=%d N=%d)",
                T, K, N);
  if (ws_bytes < b200_dense_fp8_add_rmsnorm_workspace_bytes(T, K, N))
    return fail(B200_E_WS, "b200_dense_fp8_add_rmsnorm: workspace %zu < %zu bytes", ws_bytes,
                b200_dense_fp8_add_rmsnorm_workspace_bytes(T, K, N));
  if (reinterpret_cast<uintptr_t>(ws) & 1023)
    return fail(B200_E_ALIGN, "b200_dense_fp8_add_rmsnorm: workspace must be 1024-byte aligned");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  auto up = [](size_t v) { return (v + 1023) & ~size_t(1023); };
  uint8_t* xq = static_cast<uint8_t*>(ws);
  float* xs = reinterpret_cast<float*>(xq + up(static_cast<size_t>(T < 64 ? 64 : T) * K));
  float* partials = reinterpret_cast<float*>(static_cast<uint8_t*>(ws) + b200_dense_fp8_workspace_bytes(T, K));
  CUtensorMap tmW, tmX, tmX64;
  int rc;
  if ((rc = make_tmap_bytes_2d(&tmW, w, static_cast<uint64_t>(N), K, 128, "projection weight"))) return rc;
  if ((rc = make_tmap_bytes_2d(&tmX, xq, T, K, 16, "projection activations"))) return rc;
  const bool wide = dense_wide(T, K);
  if ((rc = make_tmap_bytes_2d(&tmX64, xq, T, K, wide ? 128 : 64, "projection activations"))) return rc;
  quant_permute_f8_kernel<<<T, 256, 0, st>>>(static_cast<const bf16*>(x), T, K, 0, nullptr, 0, T, xq, xs, F8Partition{});
  F8Args a{};
  a.E_local = 1;
  a.mtiles = (N + 127) / 128;
  a.ksteps = K / 128;
  a.w_rows = N;
  a.H = K;
  a.total_rows = T;
  a.s_w = w_s;
  a.s_w_sh = w_s;
  a.a_scale = xs;
  a.status = status;
  a.kparts = proj_kparts(N, K);
  a.ksplit = proj_ksplit(N, K, T);
  a.partials = partials;
  a.nseg = 1;
  a.seg_lo[0] = 0;
  a.seg_lo[1] = N;
  a.seg_ld[0] = N;
  a.seg_out[0] = nullptr;   // not used: the sums go through `partials` (also when there is a single K part)
  const int S = a.kparts;
  const int ntiles = a.mtiles * dense_chunks(T, K) * a.ksplit;
  const int grid = ntiles < sm_count() ? ntiles : sm_count();
  launch_dense<MODE_DENSE, MODE_DENSE_W>(wide, grid, tmW, tmX, tmX64, a, st);
  add_rmsnorm_partials_kernel<<<T, 256, 0, st>>>(partials, S, T, static_cast<bf16*>(residual),
                                                 static_cast<const bf16*>(norm_w), eps, N, static_cast<bf16*>(out),
                                                 static_cast<bf16*>(proj_out));
  return launch_status("b200_dense_fp8_add_rmsnorm");
}

extern "C" int b200_add_rmsnorm(const void* proj, void* residual, const void* w, float eps, int T, int H, void* out,
                                void* stream) {
  if (!proj || !residual || !w || !out) return fail(B200_E_ARG, "b200_add_rmsnorm: null pointer");
  if (T < 0 || H <= 0 || H % 8) return fail(B200_E_ARG, "b200_add_rmsnorm: need H %% 8 == 0 (H=%d)", H);
  if (T == 0) return 0;
  add_rmsnorm_kernel<<<T, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const bf16*>(proj), static_cast<bf16*>(residual), static_cast<const bf16*>(w), eps, H,
      static_cast<bf16*>(out));
  return launch_status("b200_add_rmsnorm");
}
