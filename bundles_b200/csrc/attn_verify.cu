// Attention verify core for the gated full-attention layers: 4 draft tokens per request attend to the
// request's e4m3 KV pages and causally to each other; split-KV online softmax; output gate.
// Reference: attn_verify_kernel (qk_attn_verify.cu:354-744): S = q . k in fp32 from e4m3 operands,
// running maximum raised only when a tile exceeds it by more than 8 in the log2 domain
// (qk_attn_verify.cu:210, 264-267), P rounded to f16 before the P . V product (:297-301), split partials
// (o, m, l) merged by an ordered sum (:690-737), out = bf16(bf16(o / l) * sigmoid(gate)) (:559-562).
//
// Layout chosen for this GPU (the reference reads 1-token pages through a per-token table, :398-423):
// pages of 128 tokens; K page [kv head][128 keys][256 dims] e4m3, V page [kv head][256 dims][128 keys]
// e4m3 (dim-major, so that V arrives as the K-major B operand of the P . V product).  The 4 new tokens
// are appended to the pages by a small kernel first, and the main kernel sees them as ordinary keys
// with the causal limit key <= prefix + token.
//
// One CTA per (request, kv head, split).  S^T = K . Q^T on tcgen05 kind::f8f6f4 with the 128 keys of a
// page on the TMEM lanes and the 32 rows (4 tokens x 8 q heads) as columns, so the softmax warps own one
// key per thread; O = P . V on kind::f16 (P as the A operand: 32 real rows, the other 96 rows of the
// M = 128 tile read whatever follows P in shared memory and land in TMEM lanes nobody reads), V
// converted e4m3 -> f16 in shared memory by its own warps; the row sums are fp32 sums of the unrounded
// probabilities, as in the reference.
#include "common.cuh"
#include "host.h"

namespace b200 {

B200_DEFINE_WAIT_BUDGET_SETTER(set_wait_budget_attn_verify)

constexpr int AV_D = 256, AV_HQ = 16, AV_HKV = 2, AV_GQ = 8, AV_NT = 4, AV_ROWS = AV_GQ * AV_NT;  // 32 rows
constexpr int AV_PAGE = 128;
constexpr int AV_KTILE = AV_PAGE * AV_D;        // 32 KB e4m3: two [128 keys x 128 B] swizzled blocks
constexpr int AV_V16 = AV_D * AV_PAGE * 2;      // 64 KB f16: two [256 dims x 64 keys] swizzled blocks
constexpr int AV_PBUF = 2 * AV_ROWS * 128;      // 8 KB: two [32 rows x 64 keys] f16 blocks
constexpr int AV_QBUF = 2 * AV_ROWS * 128;      // 8 KB: two [32 rows x 128 B] e4m3 blocks
constexpr int AV_MAXPAGES = 512;                // pages of one CTA's range whose table entries are cached
constexpr int AV_SOFT = 8, AV_CONV = 8;         // softmax warps (two per TMEM quadrant), V conversion warps
constexpr int AV_THREADS = (2 + AV_SOFT + AV_CONV) * 32;  // + TMA warp + MMA warp
constexpr float AV_RESCALE_LOG2 = 8.f;
// shared memory map (bytes from the 1024-aligned base); P sits before V16 so that the A operand's rows
// 32..127 (up to 16 KB past a P block) stay inside the allocation
constexpr int AV_OFF_K = 0;                              // 2 stages
constexpr int AV_OFF_V8 = AV_OFF_K + 2 * AV_KTILE;       // 2 stages
constexpr int AV_OFF_Q = AV_OFF_V8 + 2 * AV_KTILE;
constexpr int AV_OFF_P = AV_OFF_Q + AV_QBUF;             // 2 buffers
constexpr int AV_OFF_V16 = AV_OFF_P + 2 * AV_PBUF;
constexpr int AV_OFF_BAR = AV_OFF_V16 + AV_V16;
constexpr int AV_OFF_RED = AV_OFF_BAR + 256;             // [3][4][32] floats: per-quadrant row maxima; [8][16] row sums
constexpr int AV_OFF_PT = AV_OFF_RED + (3 * 4 * 32 + 8 * 16) * 4;   // cached page-table entries
constexpr int AV_SMEM = AV_OFF_PT + AV_MAXPAGES * 4 + 1024;
// TMEM columns: O [0, 256), S double buffer [256, 288) and [288, 320)
constexpr uint32_t AV_TM_O = 0, AV_TM_S = 256;

struct AvArgs {
  const int32_t* page_table;  // [B, pt_stride]
  int pt_stride;
  const int32_t* seqlens;     // [B] tokens including the 4 drafts
  int B, splits;
  float scale_log2;
  float* part_o;              // [B * 2 * splits][32][256] unnormalised
  float* part_ml;             // [B * 2 * splits][2][32]: running maximum (log2 domain), row sum
  int32_t* status;
};

__device__ __forceinline__ void tc_mma_f16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                           uint32_t accumulate) {
  asm volatile(
      "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n" ::"r"(tmem_d),
      "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16};" ::"r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
      "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
// two e4m3 bytes (low 16 bits) -> two f16 (exact)
__device__ __forceinline__ uint32_t e4m3x2_to_f16x2(uint32_t v) {
  uint32_t r;
  asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(r) : "h"(static_cast<unsigned short>(v)));
  return r;
}
__device__ __forceinline__ unsigned short f2h_bits(float v) {
  unsigned short r;
  asm("cvt.rn.f16.f32 %0, %1;" : "=h"(r) : "f"(v));
  return r;
}
// byte offset of (row, 16-byte chunk) inside a block of 128-byte rows with the 128-byte swizzle
__device__ __forceinline__ uint32_t sw128(int row, int chunk) {
  return static_cast<uint32_t>((row >> 3) * 1024 + (row & 7) * 128 + ((chunk ^ (row & 7)) << 4));
}

constexpr uint32_t UMMA_AB_F16 = 0;

// Optional timeline of CTA 0 (compile with -DB200_TRACE): %globaltimer stamps per page of the K load issue (row 0),
// the S and P . V MMA issues (1, 2), one softmax warp's S arrival and P hand-over (3, 4), one conversion warp's
// V arrival and hand-over (5, 6); row 7: kernel start and end.
#ifdef B200_TRACE
__device__ unsigned long long g_av_trace[8][128];
#define AV_TRACE(k, i) do { if (blockIdx.x == 0 && (i) < 128) g_av_trace[k][i] = globaltimer(); } while (0)
#else
#define AV_TRACE(k, i) do { } while (0)
#endif

__global__ void __launch_bounds__(AV_THREADS, 1)
attn_verify_kernel(const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
                   const __grid_constant__ CUtensorMap tmQ, const AvArgs p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + AV_OFF_BAR);
  uint64_t* kfull = bars;          // [2] K page landed (TMA)
  uint64_t* kempty = bars + 2;     // [2] S MMAs of the page done (commit)
  uint64_t* vfull = bars + 4;      // [2] V page landed (TMA)
  uint64_t* vempty = bars + 6;     // [2] conversion warps are done with the e4m3 page
  uint64_t* sfull = bars + 8;      // [2] S^T tile complete in TMEM (commit)
  uint64_t* sfree = bars + 10;     // [2] softmax warps have read it
  uint64_t* pready = bars + 12;    // [2] P tile written (and O rescaled if needed)
  uint64_t* pvdone = bars + 14;    // [2] P . V of the tile done (commit): P buffer, V16 and O are free again
  uint64_t* v16ready = bars + 16;  // [2] f16 V half tile (keys 0..63 / 64..127) written
  uint64_t* hfree = bars + 18;     // [2] the P . V MMAs that read the half tile are done (commit)
  uint64_t* sbar = bars + 20;      // [2] the softmax warps published their row maxima (by page parity)
  uint64_t* qfull = bars + 22;     // [1] Q rows landed
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 23);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  float* redm = reinterpret_cast<float*>(smem + AV_OFF_RED);
  int32_t* spt = reinterpret_cast<int32_t*>(smem + AV_OFF_PT);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int cta = blockIdx.x;
  const int s = cta % p.splits, grp = cta / p.splits, h = grp % AV_HKV, r = grp / AV_HKV;
  if (threadIdx.x == 0) {
    for (int i = 0; i < 2; ++i) {
      mbar_init(&kfull[i], 1);
      mbar_init(&kempty[i], 1);
      mbar_init(&vfull[i], 1);
      mbar_init(&vempty[i], AV_CONV);
      mbar_init(&sfull[i], 1);
      mbar_init(&sfree[i], AV_SOFT);
      mbar_init(&pready[i], AV_SOFT);
      mbar_init(&pvdone[i], 1);
      mbar_init(&v16ready[i], AV_CONV);
      mbar_init(&hfree[i], 1);
      mbar_init(&sbar[i], AV_SOFT);
    }
    mbar_init(qfull, 1);
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmK);
    tma_prefetch_desc(&tmV);
    tma_prefetch_desc(&tmQ);
  }
  if (warp == 1) tmem_alloc(tmem_slot, 512);
  pdl_wait();
  pdl_launch();
  // this CTA's pages: tokens [0, n) of the request, n = prefix + 4 drafts, split evenly by pages
  const int n_tok = p.seqlens[r];
  const int n_prefix = n_tok - AV_NT;
  const int npages = (n_tok + AV_PAGE - 1) / AV_PAGE;
  const int pg0 = static_cast<int>(static_cast<long long>(s) * npages / p.splits);
  const int pg1 = static_cast<int>(static_cast<long long>(s + 1) * npages / p.splits);
  const int ntiles = pg1 - pg0;
  for (int i = threadIdx.x; i < ntiles && i < AV_MAXPAGES; i += AV_THREADS)
    spt[i] = p.page_table[static_cast<size_t>(r) * p.pt_stride + pg0 + i];
  fence_proxy_async();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  if (threadIdx.x == 0) AV_TRACE(7, 0);
  auto page_of = [&](int i) -> int {
    return i < AV_MAXPAGES ? spt[i] : p.page_table[static_cast<size_t>(r) * p.pt_stride + pg0 + i];
  };

  if (warp == 0) {
    // ---------------- TMA producers: lane 0 streams Q and the K pages, lane 1 the V pages.  One thread for both would
    // hold the next K page back until a V stage is free, and a V stage is free only after the page of two rounds
    // back has been converted, which waits for that page's P . V ----------------
    if (lane == 0 && ntiles > 0) {
      mbar_expect_tx(qfull, AV_QBUF);
      for (int t = 0; t < AV_NT; ++t)
        for (int c = 0; c < 2; ++c)  // the 8 q heads of this kv head for token t: one 8-row swizzle group
          tma_load_2d(smem + AV_OFF_Q + c * (AV_ROWS * 128) + t * 1024, &tmQ, c * 128,
                      (r * AV_NT + t) * AV_HQ + h * AV_GQ, qfull);
      for (int i = 0; i < ntiles; ++i) {
        const int st = i & 1;
        const uint32_t ph = (i >> 1) & 1;
        const int page = page_of(i);
        if (!mbar_wait(&kempty[st], ph ^ 1u, abort_flag, p.status, ST_WAIT_EMPTY)) break;
        AV_TRACE(0, i);
        mbar_expect_tx(&kfull[st], AV_KTILE);
        tma_load_2d(smem + AV_OFF_K + st * AV_KTILE, &tmK, 0, (page * AV_HKV + h) * AV_PAGE, &kfull[st]);
        tma_load_2d(smem + AV_OFF_K + st * AV_KTILE + AV_KTILE / 2, &tmK, 128, (page * AV_HKV + h) * AV_PAGE, &kfull[st]);
      }
    } else if (lane == 1 && ntiles > 0) {
      for (int i = 0; i < ntiles; ++i) {
        const int st = i & 1;
        const uint32_t ph = (i >> 1) & 1;
        const int page = page_of(i);
        if (!mbar_wait(&vempty[st], ph ^ 1u, abort_flag, p.status, ST_WAIT_EMPTY)) break;
        mbar_expect_tx(&vfull[st], AV_KTILE);
        tma_load_2d(smem + AV_OFF_V8 + st * AV_KTILE, &tmV, 0, (page * AV_HKV + h) * AV_D, &vfull[st]);
      }
      // the kernel's last waits (every P . V commit) cover all copies issued here
    }
  } else if (warp == 1) {
    if (lane == 0 && ntiles > 0) {  // ---------------- MMA issuer ----------------
      const uint32_t idesc_s = umma_idesc(UMMA_C_F32, UMMA_AB_E4M3, AV_ROWS);   // M = 128 keys, N = 32 rows
      // O^T = V^T . P^T: M = 128 of the 256 dims (two accumulators), N = 32 rows.  With the rows on the M side an MMA
      // would spend 128 rows' worth of tensor time on 32
      const uint32_t idesc_o = umma_idesc(UMMA_C_F32, UMMA_AB_F16, AV_ROWS);
      const uint32_t q_base = smem_u32(smem + AV_OFF_Q);
      bool ok = mbar_wait(qfull, 0, abort_flag, p.status, ST_WAIT_FULL);
      auto issue_s = [&](int j) -> bool {
        const int st = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        if (!mbar_wait(&kfull[st], ph, abort_flag, p.status, ST_WAIT_FULL)) return false;
        if (j >= 2 && !mbar_wait(&sfree[st], ph ^ 1u, abort_flag, p.status, ST_WAIT_TMEM_EMPTY)) return false;
        tc_fence_after();
        AV_TRACE(1, j);
        const uint32_t k_base = smem_u32(smem + AV_OFF_K + st * AV_KTILE);
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {  // 8 x 32 dims; dims 128..255 are the second swizzled block
          const uint32_t off = (kk >> 2) * (AV_KTILE / 2) + (kk & 3) * 32;
          const uint32_t qoff = (kk >> 2) * (AV_ROWS * 128) + (kk & 3) * 32;
          tc_mma_f8(tmem_base + AV_TM_S + st * 32, umma_desc_sw128(k_base + off), umma_desc_sw128(q_base + qoff), idesc_s,
                    kk != 0);
        }
        tc_commit(&kempty[st]);
        tc_commit(&sfull[st]);
        return true;
      };
      // the score MMAs run two pages ahead of the P . V MMAs: the softmax warps read page i + 1's scores before they
      // hand over page i's probabilities
      if (ok) ok = issue_s(0);
      if (ok && ntiles > 1) ok = issue_s(1);
      for (int i = 0; ok && i < ntiles; ++i) {
        if (i + 2 < ntiles && !issue_s(i + 2)) break;
        const int b = i & 1;
        const uint32_t ph = (i >> 1) & 1;
        if (!mbar_wait(&pready[b], ph, abort_flag, p.status, ST_WAIT_TMEM_FULL)) break;
        tc_fence_after();
        AV_TRACE(2, i);
        const uint32_t p_base = smem_u32(smem + AV_OFF_P + b * AV_PBUF);
        const uint32_t v_base = smem_u32(smem + AV_OFF_V16);
        bool good = true;
#pragma unroll
        for (int hk = 0; hk < 2; ++hk) {  // keys 0..63, then 64..127: the conversion of one half overlaps the MMAs of the other
          if (!mbar_wait(&v16ready[hk], i & 1, abort_flag, p.status, ST_WAIT_FULL)) {
            good = false;
            break;
          }
          tc_fence_after();
#pragma unroll
          for (int k4 = 0; k4 < 4; ++k4) {  // 4 x 16 keys
            const int kk = hk * 4 + k4;
            const uint64_t dp = umma_desc_sw128(p_base + hk * (AV_ROWS * 128) + k4 * 32);
            const uint32_t vb = v_base + hk * (AV_D * 128) + k4 * 32;
            tc_mma_f16(tmem_base + AV_TM_O, umma_desc_sw128(vb), dp, idesc_o, (i | kk) != 0);                    // dims 0..127
            tc_mma_f16(tmem_base + AV_TM_O + AV_ROWS, umma_desc_sw128(vb + 128 * 128), dp, idesc_o, (i | kk) != 0);  // 128..255
          }
          tc_commit(&hfree[hk]);
        }
        if (!good) break;
        tc_commit(&pvdone[b]);
      }
    }
  } else if (warp < 2 + AV_SOFT) {
    // ---------------- softmax: warps 2..9.  TMEM lane quadrant q = warp % 4 holds keys 32 q .. 32 q + 31 of the
    // page; the two warps of a quadrant take 16 of the 32 rows each.  Every warp keeps the running maximum of
    // all 32 rows (row j in lane j; identical in all warps: they read the same exchanged maxima) and its own
    // share of the row sums.  The loop is software-pipelined: the scores of page i + 1 are read and their row
    // maxima published before the probabilities of page i are formed, so neither the S MMA's completion nor
    // the exchange of the maxima is waited for where it is needed ----------------
    const int q = warp & 3, half = (warp - 2) >> 2;
    const int key_in_page = q * 32 + lane;
    float m_run = -INFINITY;  // lane j: running maximum of row j (log2 domain)
    float l_run = 0.f;        // lane l: this warp's 32 keys' share of the sum of row half*16 + (l & 15)
    bool ok = true;
    // stage A of page i: scores -> registers, masked and scaled; per-row maximum of this warp's 32 keys -> redm
    auto stage_a = [&](int i, float (&sc)[16]) -> bool {
      const int b = i & 1;
      if (!mbar_wait(&sfull[b], (i >> 1) & 1, abort_flag, p.status, ST_WAIT_TMEM_FULL)) return false;
      tc_fence_after();
      if (warp == 4 && lane == 0) AV_TRACE(3, i);
      uint32_t raw[16];
      tmem_ld16(tmem_base + AV_TM_S + b * 32 + half * 16 + (static_cast<uint32_t>(q * 32) << 16), raw);
      tmem_ld_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&sfree[b]);
      const int key = (pg0 + i) * AV_PAGE + key_in_page;  // causal limit per token: key <= prefix + token
      uint32_t mine = 0u;
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        const int tok = (half * 16 + j) >> 3;
        sc[j] = key <= n_prefix + tok ? __uint_as_float(raw[j]) * p.scale_log2 : -INFINITY;
        // order-preserving integer image of the score (NaN scores of stale keys were masked above)
        uint32_t k = __float_as_uint(sc[j]);
        k = (k & 0x80000000u) ? ~k : (k | 0x80000000u);
        const uint32_t mx = __reduce_max_sync(FULL_MASK, k);
        if (lane == j) mine = mx;
      }
      if (lane < 16) {
        const uint32_t f = (mine & 0x80000000u) ? (mine & 0x7fffffffu) : ~mine;
        redm[((i % 3) * 4 + q) * 32 + half * 16 + lane] = __uint_as_float(f);
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&sbar[b]);
      return true;
    };
    float sc_cur[16], sc_next[16];
    if (ntiles > 0) ok = stage_a(0, sc_cur);
    for (int i = 0; ok && i < ntiles; ++i) {
      const int b = i & 1;
      const uint32_t ph = (i >> 1) & 1;
      if (i + 1 < ntiles && !stage_a(i + 1, sc_next)) break;
      // stage B of page i: every warp has published its maxima
      if (!mbar_wait(&sbar[b], ph, abort_flag, p.status, ST_WAIT_STATE)) break;
      const float* rm = redm + (i % 3) * 4 * 32;
      const float tm = fmaxf(fmaxf(rm[lane], rm[32 + lane]), fmaxf(rm[64 + lane], rm[96 + lane]));
      const float m_new = tm > m_run + AV_RESCALE_LOG2 ? tm : m_run;  // -inf + 8 = -inf: the first finite maximum is taken
      const float alpha = (m_new == m_run) ? 1.f : exp2f(m_run - m_new);  // m_run = -inf gives 0
      const bool move = __any_sync(FULL_MASK, m_new != m_run);
      m_run = m_new;
      if (move) l_run *= __shfl_sync(FULL_MASK, alpha, half * 16 + (lane & 15));
      // the P buffer (and O, for a rescale) must be free: P . V of page i - 2 (same buffer) / i - 1 done
      if (i >= 2 && !mbar_wait(&pvdone[b], ph ^ 1u, abort_flag, p.status, ST_WAIT_TMEM_EMPTY)) break;
      if (move && i > 0) {
        // O^T: dims on the TMEM lanes (accumulator a holds dims 128 a + lane), rows on the columns.  This warp scales
        // the 32 lanes of its quadrant in accumulator `half`, column j by row j's alpha (held by lane j); the first
        // page overwrites O instead
        if (!mbar_wait(&pvdone[b ^ 1], ((i - 1) >> 1) & 1, abort_flag, p.status, ST_WAIT_TMEM_EMPTY)) break;
        tc_fence_after();
        for (int c = 0; c < 2; ++c) {
          const uint32_t col = AV_TM_O + half * AV_ROWS + c * 16 + (static_cast<uint32_t>(q * 32) << 16);
          uint32_t v[16];
          tmem_ld16(tmem_base + col, v);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 16; ++j)
            v[j] = __float_as_uint(__uint_as_float(v[j]) * __shfl_sync(FULL_MASK, alpha, c * 16 + j));
          tmem_st16(tmem_base + col, v);
        }
        tmem_st_wait();
        tc_fence_before();
      }
      // P^T -> shared memory as the A operand [row][key], f16, 128-byte swizzle; the row sums take the same rounded
      // probabilities (a transposing butterfly over the warp's 32 keys: lane l ends with row half*16 + (l & 15))
      uint8_t* pb = smem + AV_OFF_P + b * AV_PBUF + (key_in_page >> 6) * (AV_ROWS * 128);
      const int kb = (key_in_page & 63) * 2;  // byte of this key inside the 128-byte row
      float pf[16];
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        const int row = half * 16 + j;  // row & 7 == j & 7: the swizzle term is one of eight per-thread constants
        const float mr = __shfl_sync(FULL_MASK, m_run, row);
        // every (page, row) has at least one key inside the causal limit, so m_run is finite here and a masked
        // score (-inf) gives exactly 0; the row sums take the unrounded probabilities as the reference does
        // (qk_attn_verify.cu:290-302)
        float pv;
        asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(pv) : "f"(sc_cur[j] - mr));
        pf[j] = pv;
        *reinterpret_cast<unsigned short*>(pb + (row >> 3) * 1024 + (row & 7) * 128 + ((((kb >> 4) ^ (j & 7)) << 4) | (kb & 15))) =
            f2h_bits(pv);
      }
      fence_proxy_async();
      __syncwarp();
      if (lane == 0) mbar_arrive(&pready[b]);
      if (warp == 4 && lane == 0) AV_TRACE(4, i);
#pragma unroll
      for (int o = 8; o > 0; o >>= 1) {
        const bool up = (lane & o) != 0;
#pragma unroll
        for (int j = 0; j < o; ++j) {
          const float send = up ? pf[j] : pf[j + o];
          const float keep = up ? pf[j + o] : pf[j];
          pf[j] = keep + __shfl_xor_sync(FULL_MASK, send, o);
        }
      }
      l_run += pf[0] + __shfl_xor_sync(FULL_MASK, pf[0], 16);
#pragma unroll
      for (int j = 0; j < 16; ++j) sc_cur[j] = sc_next[j];
    }
    // ---------------- epilogue: the row sums of the eight warps meet in shared memory; every warp writes its 32 dims
    // (lanes of its quadrant in accumulator `half`) of the 32 rows of this split's partial ----------------
    float* lsum = redm + 3 * 4 * 32;  // [8 warps][16]
    if (lane < 16) lsum[(warp - 2) * 16 + lane] = l_run;
    __syncwarp();
    if (lane == 0) mbar_arrive(&sbar[ntiles & 1]);
    if (ok) {
      float* po = p.part_o + static_cast<size_t>(cta) * AV_ROWS * AV_D + half * 128 + q * 32 + lane;   // + row * AV_D
      float* pml = p.part_ml + static_cast<size_t>(cta) * 2 * AV_ROWS;
      if (ntiles == 0) {
        for (int j = 0; j < AV_ROWS; ++j) po[static_cast<size_t>(j) * AV_D] = 0.f;
        if (half == 0 && q == 0) {
          pml[lane] = -INFINITY;
          pml[AV_ROWS + lane] = 0.f;
        }
      } else {
        const int last = ntiles - 1;
        if (mbar_wait(&pvdone[last & 1], (last >> 1) & 1, abort_flag, p.status, ST_WAIT_TMEM_FULL) &&
            mbar_wait(&sbar[ntiles & 1], (ntiles >> 1) & 1, abort_flag, p.status, ST_WAIT_STATE)) {
          tc_fence_after();
          for (int c = 0; c < 2; ++c) {
            uint32_t v[16];
            tmem_ld16(tmem_base + AV_TM_O + half * AV_ROWS + c * 16 + (static_cast<uint32_t>(q * 32) << 16), v);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 16; ++j) po[static_cast<size_t>(c * 16 + j) * AV_D] = __uint_as_float(v[j]);
          }
          if (half == 0 && q == 0) {
            // row `lane`: its sum lives in the four warps of half lane / 16 (warp index = 4 * half + quadrant slot)
            const int hw = lane >> 4, j = lane & 15;
            float l = 0.f;
            for (int w = 0; w < 4; ++w) l += lsum[(hw * 4 + w) * 16 + j];
            pml[lane] = m_run;
            pml[AV_ROWS + lane] = l;
          }
        }
      }
    }
  } else {
    // ---------------- V conversion: warps 10..17.  e4m3 page [256 dims][128 keys] -> f16, same orientation, as two
    // 64-key blocks; 16 keys (one 16-byte chunk) per step ----------------
    const int ct = (warp - 2 - AV_SOFT) * 32 + lane;  // 0..255
    bool ok = true;
    for (int i = 0; ok && i < ntiles; ++i) {
      const int st = i & 1;
      const uint32_t ph = (i >> 1) & 1;
      if (!mbar_wait(&vfull[st], ph, abort_flag, p.status, ST_WAIT_FULL)) break;
      if (warp == 2 + AV_SOFT && lane == 0) AV_TRACE(5, i);
      const uint8_t* src = smem + AV_OFF_V8 + st * AV_KTILE;
      // keys past the request's last token may hold stale bytes (any bit pattern, NaN included): zero them so that
      // a zero probability times such a value cannot poison the sums
      const int keys_valid = min(AV_PAGE, n_tok - (pg0 + i) * AV_PAGE);
      for (int hk = 0; hk < 2; ++hk) {
        // the half tile is free once the MMAs of the previous page that read it are done
        if (i >= 1 && !mbar_wait(&hfree[hk], (i - 1) & 1, abort_flag, p.status, ST_WAIT_TMEM_EMPTY)) {
          ok = false;
          break;
        }
        // thread ct converts chunk c4 = ct % 4 of dim rows ct / 4 + 64 k, k = 0..3: the swizzle term depends on the
        // row modulo 8 only, so source and destination offsets advance by a constant (64 rows = 8192 bytes)
        const int c4 = ct & 3, c = hk * 4 + c4, d0 = ct >> 2;
        const uint8_t* sp = src + sw128(d0, c);
        uint8_t* dp = smem + AV_OFF_V16 + hk * (AV_D * 128) + sw128(d0, c4 * 2);
        const uint32_t hi_delta = sw128(d0, c4 * 2 + 1) - sw128(d0, c4 * 2);  // the pair's second chunk (may be negative)
        const int k0 = c * 16;
        const bool ragged = k0 + 16 > keys_valid;
        uint4 vin[4];   // the four chunks are requested before the first is converted
#pragma unroll
        for (int k = 0; k < 4; ++k) vin[k] = *reinterpret_cast<const uint4*>(sp + k * 8192);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          uint4 v = vin[k];
          if (ragged) {
            uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int e = 0; e < 16; ++e)
              if (k0 + e >= keys_valid) w[e >> 2] &= ~(0xffu << ((e & 3) * 8));
            v = make_uint4(w[0], w[1], w[2], w[3]);
          }
          uint4 lo, hi;
          lo.x = e4m3x2_to_f16x2(v.x & 0xffffu);
          lo.y = e4m3x2_to_f16x2(v.x >> 16);
          lo.z = e4m3x2_to_f16x2(v.y & 0xffffu);
          lo.w = e4m3x2_to_f16x2(v.y >> 16);
          hi.x = e4m3x2_to_f16x2(v.z & 0xffffu);
          hi.y = e4m3x2_to_f16x2(v.z >> 16);
          hi.z = e4m3x2_to_f16x2(v.w & 0xffffu);
          hi.w = e4m3x2_to_f16x2(v.w >> 16);
          *reinterpret_cast<uint4*>(dp + k * 8192) = lo;
          *reinterpret_cast<uint4*>(dp + k * 8192 + static_cast<int>(hi_delta)) = hi;
        }
        fence_proxy_async();
        __syncwarp();
        if (lane == 0) mbar_arrive(&v16ready[hk]);
      }
      if (!ok) break;
      if (lane == 0) mbar_arrive(&vempty[st]);
      if (warp == 2 + AV_SOFT && lane == 0) AV_TRACE(6, i);
    }
  }
  if (threadIdx.x == 0) AV_TRACE(7, 1);
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

// The 4 new tokens of every request go into its pages before the main kernel runs: K rows as they are, V
// transposed (one byte per dim).  One CTA per (request, token), 256 threads = dims; both kv heads.
__global__ void __launch_bounds__(256) kv_append_kernel(const uint8_t* __restrict__ k_new, const uint8_t* __restrict__ v_new,
                                                        const int32_t* __restrict__ page_table, int pt_stride,
                                                        const int32_t* __restrict__ seqlens, uint8_t* __restrict__ kcache,
                                                        uint8_t* __restrict__ vcache) {
  pdl_wait();
  pdl_launch();
  const int r = blockIdx.x / AV_NT, t = blockIdx.x % AV_NT, d = threadIdx.x;
  const int pos = seqlens[r] - AV_NT + t;
  if (pos < 0) return;
  const int page = page_table[static_cast<size_t>(r) * pt_stride + pos / AV_PAGE], in_page = pos % AV_PAGE;
  const size_t tok = static_cast<size_t>(r) * AV_NT + t;
  for (int h = 0; h < AV_HKV; ++h) {
    const size_t ph = static_cast<size_t>(page) * AV_HKV + h;
    kcache[(ph * AV_PAGE + in_page) * AV_D + d] = k_new[(tok * AV_HKV + h) * AV_D + d];
    vcache[(ph * AV_D + d) * AV_PAGE + in_page] = v_new[(tok * AV_HKV + h) * AV_D + d];
  }
}

// Merge of the split partials and the output gate: per (request, kv head, row) the splits are added in split order
// with weights 2^(m_s - M); out = bf16(bf16(o / l) * sigmoid(gate)).  One CTA per (group, token, q head of the group),
// 256 threads = dims; every load of a row's splits is issued before the first is used (one dependent round trip per
// row instead of two per split).
constexpr int AV_MAXS = 64;
__global__ void __launch_bounds__(256) attn_combine_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                                           const bf16* __restrict__ gate, int splits,
                                                           bf16* __restrict__ out) {
  __shared__ float s_m[AV_MAXS], s_l[AV_MAXS];
  pdl_wait();
  pdl_launch();
  const int g = blockIdx.x % AV_GQ, t = (blockIdx.x / AV_GQ) % AV_NT, grp = blockIdx.x / (AV_GQ * AV_NT);
  const int d = threadIdx.x;
  const int h = grp % AV_HKV, r = grp / AV_HKV;
  const int row = t * AV_GQ + g;
  const size_t c0 = static_cast<size_t>(grp) * splits;
  if (d < splits) {
    s_m[d] = part_ml[(c0 + d) * 2 * AV_ROWS + row];
    s_l[d] = part_ml[(c0 + d) * 2 * AV_ROWS + AV_ROWS + row];
  }
  const size_t o = (static_cast<size_t>(r) * AV_NT + t) * (AV_HQ * AV_D) + static_cast<size_t>(h * AV_GQ + g) * AV_D + d;
  const float gv = bf2f(gate[o]);
  float num = 0.f, den = 0.f, M = -INFINITY;
  // the partial rows of up to 8 splits at a time are in flight together
  for (int s0 = 0; s0 < splits; s0 += 8) {
    float po[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) po[u] = s0 + u < splits ? part_o[((c0 + s0 + u) * AV_ROWS + row) * AV_D + d] : 0.f;
    if (s0 == 0) {
      __syncthreads();
      for (int s = 0; s < splits; ++s) M = fmaxf(M, s_m[s]);
    }
#pragma unroll
    for (int u = 0; u < 8; ++u)
      if (s0 + u < splits) {
        const float m = s_m[s0 + u];
        const float w = m == -INFINITY ? 0.f : exp2f(m - M);
        num = fmaf(po[u], w, num);
        den = fmaf(s_l[s0 + u], w, den);
      }
  }
  out[o] = f2bf(rbf(num / den) * (1.f / (1.f + __expf(-gv))));
}

}  // namespace b200

using namespace b200;

#ifdef B200_TRACE
extern "C" int b200_av_trace_read(unsigned long long* host) {
  return static_cast<int>(cudaMemcpyFromSymbol(host, g_av_trace, sizeof(g_av_trace)));
}
#endif

extern "C" int b200_attn_verify_splits(int B) {
  if (B <= 0) return 0;
  int s = sm_count() / (B * AV_HKV);
  return s < 1 ? 1 : (s > 16 ? 16 : s);
}

extern "C" size_t b200_attn_verify_workspace_bytes(int B, int splits) {
  if (B <= 0 || splits <= 0) return 0;
  const size_t ctas = static_cast<size_t>(B) * AV_HKV * splits;
  return ctas * AV_ROWS * AV_D * 4 + ctas * 2 * AV_ROWS * 4;
}

extern "C" int b200_attn_verify(const void* q, const void* gate, const void* k_new, const void* v_new, void* kcache,
                                void* vcache, int num_pages, const int32_t* page_table, int pt_stride,
                                const int32_t* seqlens, int B, float scale, int splits, void* out, void* ws,
                                size_t ws_bytes, int32_t* status, void* stream) {
  if (!q || !gate || !k_new || !v_new || !kcache || !vcache || !page_table || !seqlens || !out || !ws)
    return fail(B200_E_ARG, "b200_attn_verify: null pointer");
  if (B <= 0 || num_pages <= 0 || pt_stride <= 0 || splits <= 0 || splits > 64)
    return fail(B200_E_ARG, "b200_attn_verify: need B, num_pages, pt_stride >= 1 and 1 <= splits <= 64 (B=%d splits=%d)", B,
                splits);
  if (ws_bytes < b200_attn_verify_workspace_bytes(B, splits))
    return fail(B200_E_WS, "b200_attn_verify: workspace %zu < %zu bytes", ws_bytes,
                b200_attn_verify_workspace_bytes(B, splits));
  if ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(kcache) | reinterpret_cast<uintptr_t>(vcache) |
       reinterpret_cast<uintptr_t>(ws)) & 15)
    return fail(B200_E_ALIGN, "b200_attn_verify: q, caches and workspace must be 16-byte aligned");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  CUtensorMap tmK, tmV, tmQ;
  int rc;
  if ((rc = make_tmap_bytes_2d(&tmK, kcache, static_cast<uint64_t>(num_pages) * AV_HKV * AV_PAGE, AV_D, 128, "k cache")))
    return rc;
  if ((rc = make_tmap_bytes_2d(&tmV, vcache, static_cast<uint64_t>(num_pages) * AV_HKV * AV_D, AV_PAGE, 256, "v cache")))
    return rc;
  if ((rc = make_tmap_bytes_2d(&tmQ, q, static_cast<uint64_t>(B) * AV_NT * AV_HQ, AV_D, 8, "q"))) return rc;
  static DeviceOnce once;
  once.run([] { cudaFuncSetAttribute(attn_verify_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, AV_SMEM); });
  launch_k(kv_append_kernel, dim3(B * AV_NT), dim3(256), 0, st, static_cast<const uint8_t*>(k_new),
           static_cast<const uint8_t*>(v_new), page_table, pt_stride, seqlens, static_cast<uint8_t*>(kcache),
           static_cast<uint8_t*>(vcache));
  AvArgs a{};
  a.page_table = page_table;
  a.pt_stride = pt_stride;
  a.seqlens = seqlens;
  a.B = B;
  a.splits = splits;
  a.scale_log2 = scale * 1.4426950408889634f;
  a.part_o = static_cast<float*>(ws);
  a.part_ml = a.part_o + static_cast<size_t>(B) * AV_HKV * splits * AV_ROWS * AV_D;
  a.status = status;
  launch_k(attn_verify_kernel, dim3(B * AV_HKV * splits), dim3(AV_THREADS), AV_SMEM, st, tmK, tmV, tmQ, a);
  launch_k(attn_combine_kernel, dim3(B * AV_HKV * AV_NT * AV_GQ), dim3(256), 0, st, static_cast<const float*>(a.part_o),
           static_cast<const float*>(a.part_ml), static_cast<const bf16*>(gate), splits, static_cast<bf16*>(out));
  return launch_status("b200_attn_verify");
}
