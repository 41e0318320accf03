// MoE block in fp8 e4m3 with 128 x 128 weight block scales and per-(token, 128-channel) activation
// scales: activation quantise + permute, grouped GEMMs on tcgen05 (kind::f8f6f4), SwiGLU / unpermute
// epilogues.  The reference has no block-scaled fp8 MoE; the structure follows its int8 twin
// (qk_moe_prefill_i8.cu:3649-3651, 3905-3945): per 128-k block the MMA chain starts from zero in a
// TMEM partial buffer and is promoted by the epilogue warps, acc = fma(partial, a_scale * w_scale,
// acc), with two partial buffers so that block g + 1's MMAs overlap block g's promotion.
//
// Orientation as in the int8 kernels: M = 128 weight rows (exactly one weight scale block row),
// N = 16..64 tokens of one expert, K = 32 bytes per MMA; weights and expert-sorted token rows arrive
// by 2-D TMA with the 128-byte swizzle.  Final accumulators live in registers (2 x 64 fp32 per thread
// for gate and up), which is what limits N to 64 here.
#include "common.cuh"
#include "host.h"

namespace b200 {

constexpr int F8_TILE = 128 * 128;       // weight tile bytes per stage
constexpr int F8_BTILE = 64 * 128;       // token tile bytes per stage (<= 64 rows)
constexpr int F8_THREADS = 320;          // TMA warp, MMA warp, 8 epilogue warps (two per TMEM lane quadrant)
constexpr int F8_MAXKG = 32;             // k blocks per row of scales held in shared memory (K <= 4096)

// ---- activation quantisers ----------------------------------------------------------------------------
// scale = max(amax / 448, 1e-12), y = e4m3(x * (1 / scale)) per (row, 128-channel group): fp8.py:21-34.
__device__ __forceinline__ uint2 quant8_e4m3(const uint4 v, float inv) {
  return make_uint2(e4m3x4(bf_lo(v.x) * inv, bf_hi(v.x) * inv, bf_lo(v.y) * inv, bf_hi(v.y) * inv),
                    e4m3x4(bf_lo(v.z) * inv, bf_hi(v.z) * inv, bf_lo(v.w) * inv, bf_hi(v.w) * inv));
}
__device__ __forceinline__ float amax8(const uint4 v) {
  float a = fmaxf(fmaxf(fabsf(bf_lo(v.x)), fabsf(bf_hi(v.x))), fmaxf(fabsf(bf_lo(v.y)), fabsf(bf_hi(v.y))));
  return fmaxf(a, fmaxf(fmaxf(fabsf(bf_lo(v.z)), fabsf(bf_hi(v.z))), fmaxf(fabsf(bf_lo(v.w)), fabsf(bf_hi(v.w)))));
}

// one CTA per token; 16 consecutive threads own one 128-channel group (8 channels each)
__global__ void __launch_bounds__(256) quant_permute_f8_kernel(const bf16* __restrict__ x, int T, int H, int K,
                                                               const int32_t* __restrict__ row_of_pair,
                                                               int with_shared, uint8_t* __restrict__ xq,
                                                               float* __restrict__ xs) {
  __shared__ int rows[40];
  const int t = blockIdx.x, tid = threadIdx.x;
  if (tid < K) rows[tid] = row_of_pair[t * K + tid];
  if (tid == K) rows[K] = with_shared ? T * K + t : -1;
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
};

constexpr int MODE_DOWN = 0, MODE_UP = 1, MODE_LM = 2, MODE_DENSE = 3;

template <int MODE>
struct F8Cfg {
  static constexpr bool UP = MODE == MODE_UP;
  static constexpr int NA = UP ? 2 : 1;
  static constexpr int STAGE = NA * F8_TILE + F8_BTILE;
  static constexpr int STAGES = UP ? 4 : 6;
  static constexpr int META = 8 * (32 * F8_MAXKG * 4 + 32 * 8);  // per epilogue warp: scales, slot, weight of its 32 columns
  static constexpr int SMEM = STAGES * STAGE + 1024 + 256 + META;
  static constexpr int TMEM = UP ? 256 : 128;
};

template <int MODE>
__global__ void __launch_bounds__(F8_THREADS, 1)
moe_gemm_f8_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmWsh,
                   const __grid_constant__ CUtensorMap tmX, const F8Args p) {
  using C = F8Cfg<MODE>;
  constexpr bool UP = MODE == MODE_UP, LM = MODE == MODE_LM || MODE == MODE_DENSE, DENSE = MODE == MODE_DENSE;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + C::STAGES * C::STAGE);
  uint64_t* empty = full + C::STAGES;
  uint64_t* pfull = empty + C::STAGES;   // [2] a 128-k partial is complete in TMEM
  uint64_t* pempty = pfull + 2;          // [2] the epilogue warps have promoted it
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(pempty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  uint8_t* meta = smem + C::STAGES * C::STAGE + 256;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int s = 0; s < C::STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&pfull[b], 1);
      mbar_init(&pempty[b], 8);
    }
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmW);
    tma_prefetch_desc(&tmWsh);
    tma_prefetch_desc(&tmX);
  }
  if (warp == 1) tmem_alloc(tmem_slot, C::TMEM);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const int ntiles = LM ? p.mtiles : p.L.nblocks[0] * p.mtiles;

  auto decode = [&](int tile, int& e, int& row0, int& n, int& mt) -> bool {
    if (LM) {  // dense: every tile is 128 vocabulary rows against all the tokens
      e = 0;
      row0 = 0;
      n = p.total_rows;
      mt = tile;
      return n >= 1 && n <= 64;
    }
    const int blk = tile / p.mtiles;
    mt = tile - blk * p.mtiles;
    e = p.L.blk_expert[blk];
    row0 = p.L.blk_row0[blk];
    n = p.L.blk_rows[blk];
    return e >= 0 && e <= p.E_local && n >= 1 && n <= 64 && row0 >= 0 && row0 + n <= p.total_rows;
  };

  if (warp == 0) {
    if (lane == 0) {  // ---------------- TMA producer ----------------
      int stage = 0, issued = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; ok && tile < ntiles; tile += gridDim.x) {
        int e, row0, n, mt;
        if (!decode(tile, e, row0, n, mt)) continue;
        const int nb16 = (n + 15) >> 4;
        const CUtensorMap* mapW = (e == p.E_local) ? &tmWsh : &tmW;
        const int wrow = (e == p.E_local ? 0 : e * p.w_rows) + mt * 128;
        for (int ks = 0; ks < p.ksteps; ++ks) {
          if (!mbar_wait(&empty[stage], phase ^ 1u, abort_flag, p.status, ST_WAIT_EMPTY)) {
            ok = false;
            break;
          }
          uint8_t* sA = smem + stage * C::STAGE;
          uint8_t* sB = sA + C::NA * F8_TILE;
          mbar_expect_tx(&full[stage], C::NA * F8_TILE + nb16 * 2048);
          tma_load_2d(sA, mapW, ks * 128, wrow, &full[stage]);
          if (UP) tma_load_2d(sA + F8_TILE, mapW, ks * 128, wrow + p.I, &full[stage]);
          for (int b = 0; b < nb16; ++b) tma_load_2d(sB + b * 2048, &tmX, ks * 128, row0 + 16 * b, &full[stage]);
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
      for (int tile = blockIdx.x; ok && tile < ntiles; tile += gridDim.x) {
        int e, row0, n, mt;
        if (!decode(tile, e, row0, n, mt)) continue;
        const uint32_t N = static_cast<uint32_t>((n + 15) & ~15);
        const uint32_t idesc = umma_idesc(UMMA_C_F32, UMMA_AB_E4M3, N);
        for (int ks = 0; ks < p.ksteps && ok; ++ks, ++g) {
          const uint32_t pb = g & 1u, pphase = (g >> 1) & 1u;
          if (!mbar_wait(&pempty[pb], pphase ^ 1u, abort_flag, p.status, ST_WAIT_TMEM_EMPTY) ||
              !mbar_wait(&full[stage], phase, abort_flag, p.status, ST_WAIT_FULL)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sA = smem_u32(smem + stage * C::STAGE);
          const uint32_t sB = sA + C::NA * F8_TILE;
          const uint32_t d0 = tmem_base + pb * (UP ? 128 : 64);
#pragma unroll
          for (int kk = 0; kk < 4; ++kk) {
            const uint64_t db = umma_desc_sw128(sB + kk * 32);
            tc_mma_f8(d0, umma_desc_sw128(sA + kk * 32), db, idesc, kk != 0);
            if (UP) tc_mma_f8(d0 + 64, umma_desc_sw128(sA + F8_TILE + kk * 32), db, idesc, kk != 0);
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
    // ---------------- promotion + epilogue: warps 2..9.  TMEM lane quadrant = warp % 4; the two warps of a
    // quadrant share a scheduler and take alternate 16-column chunks (chunk index parity = `half`), so each
    // thread keeps at most 32 (+32 for up) accumulators ----------------
    const int q = warp & 3;
    const int half = (warp - 2) >> 2;
    float* m_as = reinterpret_cast<float*>(meta + (warp - 2) * (32 * F8_MAXKG * 4 + 32 * 8));  // [32][ksteps]
    float* m_wt = m_as + 32 * F8_MAXKG;                                                         // [32]
    int* m_slot = reinterpret_cast<int*>(m_wt + 32);                                            // [32]
    const float* __restrict__ a_scale = p.a_scale;
    uint32_t g = 0;
    bool ok = true;
    // local column l (0..31) of this warp is tile column col(l) = (l / 16) * 32 + half * 16 + l % 16
    for (int tile = blockIdx.x; ok && tile < ntiles; tile += gridDim.x) {
      int e, row0, n, mt;
      if (!decode(tile, e, row0, n, mt)) {
        if (lane == 0 && p.status) atomicCAS(p.status, 0, ST_BAD_LIST);
        continue;
      }
      __syncwarp();
      for (int i = lane; i < 32 * p.ksteps; i += 32) {
        const int l = i / p.ksteps, ks = i - l * p.ksteps;
        const int c = (l >> 4) * 32 + half * 16 + (l & 15);
        m_as[i] = c < n ? a_scale[static_cast<size_t>(row0 + c) * p.ksteps + ks] : 0.f;
      }
      {
        const int c = (lane >> 4) * 32 + half * 16 + (lane & 15);
        int slot = -1;
        float wt = 0.f;
        if (!LM && c < n) {
          slot = p.L.slot_of_row[row0 + c];
          wt = p.L.wt_of_row[row0 + c];
          if (slot >= p.total_rows) slot = -1;
        }
        m_slot[lane] = slot;
        m_wt[lane] = wt;
      }
      __syncwarp();
      const bool shared_e = (e == p.E_local);
      const float* swb = shared_e ? p.s_w_sh : p.s_w + static_cast<size_t>(e) * (p.w_rows / 128) * p.ksteps;
      const float* sw_a = swb + static_cast<size_t>(mt) * p.ksteps;                      // gate / down block row
      const float* sw_b = swb + static_cast<size_t>(p.I / 128 + mt) * p.ksteps;          // up block row (UP only)
      float acc_a[32], acc_b[UP ? 32 : 1];
#pragma unroll
      for (int c = 0; c < 32; ++c) acc_a[c] = 0.f;
      if (UP)
#pragma unroll
        for (int c = 0; c < 32; ++c) acc_b[c] = 0.f;
      for (int ks = 0; ks < p.ksteps; ++ks, ++g) {
        const uint32_t pb = g & 1u, pphase = (g >> 1) & 1u;
        const float wsa = __ldg(sw_a + ks), wsb = UP ? __ldg(sw_b + ks) : 0.f;
        if (!mbar_wait(&pfull[pb], pphase, abort_flag, p.status, ST_WAIT_TMEM_FULL)) {
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t taddr = tmem_base + pb * (UP ? 128 : 64) + half * 16 + (static_cast<uint32_t>(q * 32) << 16);
#pragma unroll
        for (int h2 = 0; h2 < 2; ++h2) {
          if (h2 * 32 + half * 16 < n) {
            uint32_t ra[16], rb[16];
            tmem_ld16(taddr + h2 * 32, ra);
            if (UP) tmem_ld16(taddr + 64 + h2 * 32, rb);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 16; ++i) {
              const float as = m_as[(h2 * 16 + i) * p.ksteps + ks];
              acc_a[h2 * 16 + i] = __fmaf_rn(__uint_as_float(ra[i]), __fmul_rn(as, wsa), acc_a[h2 * 16 + i]);
              if (UP) acc_b[h2 * 16 + i] = __fmaf_rn(__uint_as_float(rb[i]), __fmul_rn(as, wsb), acc_b[h2 * 16 + i]);
            }
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&pempty[pb]);
      }
      if (!ok) break;
      const int r = mt * 128 + q * 32 + lane;
      if (DENSE) {
        // plain projection: out[token][feature] = bf16(acc)
        if (r < p.w_rows) {
          bf16* __restrict__ o = p.h_out + r;
#pragma unroll
          for (int l = 0; l < 32; ++l) {
            const int c = (l >> 4) * 32 + half * 16 + (l & 15);
            if (c < n) o[static_cast<size_t>(c) * p.w_rows] = f2bf(acc_a[l]);
          }
        }
      } else if (LM) {
        // per token: the largest logit of this warp's 32 vocabulary rows and its id (ties to the lower
        // id) as one packed 64-bit key per (tile, quadrant, token); a small kernel takes the max over them
        const bool live = r < p.w_rows;
#pragma unroll
        for (int l = 0; l < 32; ++l) {
          const int c = (l >> 4) * 32 + half * 16 + (l & 15);
          if (c < n) {
            const float v = acc_a[l];
            if (p.lm_logits && live) p.lm_logits[static_cast<size_t>(c) * p.w_rows + r] = v;
            uint32_t key = 0u;
            if (live && v == v) {
              const float vz = v + 0.f;
              key = __float_as_uint(vz);
              key = (key & 0x80000000u) ? ~key : (key | 0x80000000u);
              if (key < 2u) key = 2u;
            } else if (live) {
              key = 1u;
            }
            const uint32_t m = __reduce_max_sync(FULL_MASK, key);
            const uint32_t id = __reduce_min_sync(FULL_MASK, (key == m && live) ? static_cast<uint32_t>(r) : 0xffffffffu);
            if (lane == 0)
              p.lm_keys[(static_cast<size_t>(tile) * 4 + q) * n + c] =
                  m == 0u ? 0ull
                          : (static_cast<unsigned long long>(m) << 32) |
                                (0xffffffffu - static_cast<uint32_t>(p.lm_shard_lo + static_cast<int>(id)));
          }
        }
      } else if (UP) {
        bf16* __restrict__ hout = p.h_out + static_cast<size_t>(row0) * p.I + r;
#pragma unroll
        for (int l = 0; l < 32; ++l) {
          const int c = (l >> 4) * 32 + half * 16 + (l & 15);
          if (c < n) {
            const float gv = rbf(acc_a[l]), uv = rbf(acc_b[l]);
            const bf16 hv = f2bf(__fmul_rn(__fdiv_rn(gv, 1.f + __expf(-gv)), uv));
            hout[static_cast<size_t>(c) * p.I] = hv;
            if (p.dbg_h && m_slot[l] >= 0) p.dbg_h[static_cast<size_t>(m_slot[l]) * p.I + r] = hv;
          }
        }
      } else {
        bf16* __restrict__ cache = p.cache + r;
#pragma unroll
        for (int l = 0; l < 32; ++l) {
          const int c = (l >> 4) * 32 + half * 16 + (l & 15);
          if (c < n && m_slot[l] >= 0) cache[static_cast<size_t>(m_slot[l]) * p.H] = f2bf(__fmul_rn(acc_a[l], m_wt[l]));
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, C::TMEM);
  }
}

// x bf16 [T, H] -> e4m3 rows [T, H] + scales [T, H/128] in token order (no permutation)
void b200_quant_rows_f8_launch(const void* x, int T, int H, uint8_t* xq, float* xs, cudaStream_t st) {
  quant_permute_f8_kernel<<<T, 256, 0, st>>>(static_cast<const bf16*>(x), T, H, 0, nullptr, 1, xq, xs);
}

struct F8Layout {
  size_t xq, xs, h, hq, hs, total;
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
  l.total = o;
  return l;
}

}  // namespace b200

using namespace b200;

extern "C" size_t b200_moe_fp8_workspace_bytes(int T, int H, int I, int K) {
  if (T <= 0 || H <= 0 || I <= 0 || K <= 0) return 0;
  return f8_layout(T, H, I, K).total;
}

extern "C" int b200_moe_fp8(const void* x, int T, int H, int I, int K, int E_local, const b200_moe_weights* w,
                            const b200_moe_lists* lists, void* cache, void* ws, size_t ws_bytes, void* dbg_h,
                            int stages, int32_t* status, void* stream) {
  if (!x || !w || !lists || !cache || !ws || !w->w13 || !w->s13 || !w->w2 || !w->s2)
    return fail(B200_E_ARG, "b200_moe_fp8: null pointer");
  if (T <= 0 || K <= 0 || K > 32 || E_local <= 0 || H % 128 || I % 128 || H <= 0 || I <= 0 || H / 128 > F8_MAXKG ||
      I / 128 > F8_MAXKG)
    return fail(B200_E_ARG, "b200_moe_fp8: need H, I multiples of 128 and <= 4096, 1 <= K <= 32 (T=%d H=%d I=%d K=%d)",
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
  CUtensorMap tmW13, tmSh13, tmXq, tmW2, tmSh2, tmHq;
  int rc;
  if ((rc = make_tmap_bytes_2d(&tmW13, w->w13, static_cast<uint64_t>(E_local) * 2 * I, H, 128, "w13"))) return rc;
  if ((rc = make_tmap_bytes_2d(&tmSh13, shared ? w->sh13 : w->w13, 2 * I, H, 128, "sh13"))) return rc;
  if ((rc = make_tmap_bytes_2d(&tmXq, xq, rows, H, 16, "xq"))) return rc;
  if ((rc = make_tmap_bytes_2d(&tmW2, w->w2, static_cast<uint64_t>(E_local) * H, I, 128, "w2"))) return rc;
  if ((rc = make_tmap_bytes_2d(&tmSh2, shared ? w->sh2 : w->w2, H, I, 128, "sh2"))) return rc;
  if ((rc = make_tmap_bytes_2d(&tmHq, hq, rows, I, 16, "hq"))) return rc;
  static bool attr_done[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !attr_done[dev]) {
    cudaFuncSetAttribute(moe_gemm_f8_kernel<MODE_UP>, cudaFuncAttributeMaxDynamicSharedMemorySize, F8Cfg<MODE_UP>::SMEM);
    cudaFuncSetAttribute(moe_gemm_f8_kernel<MODE_DOWN>, cudaFuncAttributeMaxDynamicSharedMemorySize, F8Cfg<MODE_DOWN>::SMEM);
    attr_done[dev] = true;
  }
  if (stages == 0) stages = 15;
  if (stages & B200_MOE_STAGE_QUANT)
    quant_permute_f8_kernel<<<T, 256, 0, st>>>(static_cast<const bf16*>(x), T, H, K, L.row_of_pair, shared ? 1 : 0, xq, xs);
  F8Args a{};
  a.L = L;
  a.E_local = E_local;
  a.I = I;
  a.H = H;
  a.total_rows = rows;
  a.status = status;
  const int grid = sm_count();
  a.mtiles = I / 128;
  a.ksteps = H / 128;
  a.w_rows = 2 * I;
  a.s_w = w->s13;
  a.s_w_sh = w->shs13;
  a.a_scale = xs;
  a.h_out = h;
  a.dbg_h = static_cast<bf16*>(dbg_h);
  if (stages & B200_MOE_STAGE_UP)
    moe_gemm_f8_kernel<MODE_UP><<<grid, F8_THREADS, F8Cfg<MODE_UP>::SMEM, st>>>(tmW13, tmSh13, tmXq, a);
  if (stages & B200_MOE_STAGE_HQUANT)
    quant_rows_f8_kernel<<<(rows + 7) / 8, 256, 0, st>>>(h, rows, I, L.slot_of_row, hq, hs);
  a.mtiles = H / 128;
  a.ksteps = I / 128;
  a.w_rows = H;
  a.s_w = w->s2;
  a.s_w_sh = w->shs2;
  a.a_scale = hs;
  a.h_out = nullptr;
  a.cache = static_cast<bf16*>(cache);
  a.dbg_h = nullptr;
  if (stages & B200_MOE_STAGE_DOWN)
    moe_gemm_f8_kernel<MODE_DOWN><<<grid, F8_THREADS, F8Cfg<MODE_DOWN>::SMEM, st>>>(tmW2, tmSh2, tmHq, a);
  return launch_status("b200_moe_fp8");
}

// ---- LM head shard with fused argmax ------------------------------------------------------------------
namespace b200 {
__global__ void lmhead_finish_kernel(const unsigned long long* __restrict__ keys, int parts, int T,
                                     float* __restrict__ max_out, int32_t* __restrict__ idx_out) {
  // one warp per token: max over the (tile, warp) partial keys
  const int t = blockIdx.x, lane = threadIdx.x;
  unsigned long long k = 0ull;
  for (int i = lane; i < parts; i += 32) {
    const unsigned long long v = keys[static_cast<size_t>(i) * T + t];
    k = v > k ? v : k;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const unsigned long long v = __shfl_xor_sync(FULL_MASK, k, o);
    k = v > k ? v : k;
  }
  if (lane != 0) return;
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
static LmLayout lm_layout(int T, int H, int V_shard) {
  auto up = [](size_t v) { return (v + 1023) & ~size_t(1023); };
  LmLayout l;
  size_t o = 0;
  l.xq = o; o = up(o + static_cast<size_t>(64) * H);  // 64 rows so that every 16-row TMA box is in bounds
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
  if (T <= 0 || T > 64 || H <= 0 || H % 128 || H / 128 > F8_MAXKG || V_shard <= 0 || shard_lo < 0)
    return fail(B200_E_ARG, "b200_lmhead_argmax: need 1 <= T <= 64, H %% 128 == 0, H <= 4096 (T=%d H=%d V=%d)", T, H,
                V_shard);
  const LmLayout l = lm_layout(T, H, V_shard);
  if (ws_bytes < l.total) return fail(B200_E_WS, "b200_lmhead_argmax: workspace %zu < %zu bytes", ws_bytes, l.total);
  if (reinterpret_cast<uintptr_t>(ws) & 1023) return fail(B200_E_ALIGN, "b200_lmhead_argmax: workspace must be 1024-byte aligned");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  uint8_t* base = static_cast<uint8_t*>(ws);
  uint8_t* xq = base + l.xq;
  float* xs = reinterpret_cast<float*>(base + l.xs);
  unsigned long long* keys = reinterpret_cast<unsigned long long*>(base + l.keys);
  CUtensorMap tmW, tmX;
  int rc;
  if ((rc = make_tmap_bytes_2d(&tmW, w, static_cast<uint64_t>(V_shard), H, 128, "lm_head weight"))) return rc;
  if ((rc = make_tmap_bytes_2d(&tmX, xq, T, H, 16, "lm_head activations"))) return rc;
  static bool attr_done[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !attr_done[dev]) {
    cudaFuncSetAttribute(moe_gemm_f8_kernel<MODE_LM>, cudaFuncAttributeMaxDynamicSharedMemorySize, F8Cfg<MODE_LM>::SMEM);
    attr_done[dev] = true;
  }
  // K = 0 routed picks: the "shared expert" row of token t is row t
  quant_permute_f8_kernel<<<T, 256, 0, st>>>(static_cast<const bf16*>(x), T, H, 0, nullptr, 1, xq, xs);
  F8Args a{};
  a.E_local = 1;
  a.mtiles = (V_shard + 127) / 128;
  a.ksteps = H / 128;
  a.w_rows = V_shard;
  a.I = 0;
  a.H = H;
  a.total_rows = T;
  a.s_w = w_s;
  a.s_w_sh = w_s;
  a.a_scale = xs;
  a.status = status;
  a.lm_keys = keys;
  a.lm_logits = logits_out;
  a.lm_shard_lo = shard_lo;
  const int grid = a.mtiles < sm_count() ? a.mtiles : sm_count();
  moe_gemm_f8_kernel<MODE_LM><<<grid, F8_THREADS, F8Cfg<MODE_LM>::SMEM, st>>>(tmW, tmW, tmX, a);
  lmhead_finish_kernel<<<T, 32, 0, st>>>(keys, a.mtiles * 4, T, max_out, idx_out);
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
  return up(static_cast<size_t>(64) * H) + up(static_cast<size_t>(T) * (H / 128) * 4);
}

extern "C" int b200_dense_fp8(const void* x, int T, int H, const void* w, const float* w_s, int N, void* out, void* ws,
                              size_t ws_bytes, int32_t* status, void* stream) {
  if (!x || !w || !w_s || !out || !ws) return fail(B200_E_ARG, "b200_dense_fp8: null pointer");
  if (T <= 0 || T > 64 || H <= 0 || H % 128 || H / 128 > F8_MAXKG || N <= 0)
    return fail(B200_E_ARG, "b200_dense_fp8: need 1 <= T <= 64, H %% 128 == 0, H <= 4096 (T=%d H=%d N=%d)", T, H, N);
  if (ws_bytes < b200_dense_fp8_workspace_bytes(T, H))
    return fail(B200_E_WS, "b200_dense_fp8: workspace %zu < %zu bytes", ws_bytes, b200_dense_fp8_workspace_bytes(T, H));
  if (reinterpret_cast<uintptr_t>(ws) & 1023) return fail(B200_E_ALIGN, "b200_dense_fp8: workspace must be 1024-byte aligned");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  uint8_t* xq = static_cast<uint8_t*>(ws);
  float* xs = reinterpret_cast<float*>(xq + ((static_cast<size_t>(64) * H + 1023) & ~size_t(1023)));
  CUtensorMap tmW, tmX;
  int rc;
  if ((rc = make_tmap_bytes_2d(&tmW, w, static_cast<uint64_t>(N), H, 128, "dense weight"))) return rc;
  if ((rc = make_tmap_bytes_2d(&tmX, xq, T, H, 16, "dense activations"))) return rc;
  static bool attr_done[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !attr_done[dev]) {
    cudaFuncSetAttribute(moe_gemm_f8_kernel<MODE_DENSE>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                         F8Cfg<MODE_DENSE>::SMEM);
    attr_done[dev] = true;
  }
  quant_permute_f8_kernel<<<T, 256, 0, st>>>(static_cast<const bf16*>(x), T, H, 0, nullptr, 1, xq, xs);
  F8Args a{};
  a.E_local = 1;
  a.mtiles = (N + 127) / 128;
  a.ksteps = H / 128;
  a.w_rows = N;
  a.H = H;
  a.total_rows = T;
  a.s_w = w_s;
  a.s_w_sh = w_s;
  a.a_scale = xs;
  a.h_out = static_cast<bf16*>(out);
  a.status = status;
  const int grid = a.mtiles < sm_count() ? a.mtiles : sm_count();
  moe_gemm_f8_kernel<MODE_DENSE><<<grid, F8_THREADS, F8Cfg<MODE_DENSE>::SMEM, st>>>(tmW, tmW, tmX, a);
  return launch_status("b200_dense_fp8");
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
