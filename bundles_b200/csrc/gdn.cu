// Gated DeltaNet speculative verify: conv + SiLU, q/k L2 norm, gates, delta-rule recurrence over
// the 4 draft tokens in closed form, gated RMSNorm; then either the explicit state / conv-state write-back
// at the accepted length, or the appends to the reference engine's (d, k, g) ring.
//
// Replaces qk_gdn_verify.cu:293 gdn_verify_kernel (host glue gdn_fused.py:37-57).
// The window algebra is the reference's (qk_gdn_verify.cu:633-762):
//   hq_s = S q_s, hk_s = S k_s;  R_s = beta_s (v_s - e^{G_s} hk_s);  D = (I + A)^-1 R with
//   A_ij = beta_i e^{G_i - G_j} k_i.k_j (i > j);  o_s = e^{G_s} hq_s + sum_{i<=s} D_i e^{G_s - G_i} k_i.q_s;
//   S_n = e^{G_{n-1}} S + sum_{i<n} e^{G_{n-1} - G_i} D_i k_i^T.
// The 128 x 128 x 8 products S [q | k] run on the tensor core in tf32 (tcgen05.mma kind::tf32 straight
// from the swizzled state tile in shared memory, accumulators in TMEM), the reference's precision for
// these dots (TF32 mma.sync, qk_gdn_verify.cu:173-179); everything else is fp32.
//
// Two state layouts (template parameter REPLAY of both kernels):
//  * explicit state (b200_gdn_verify): a unit reads its 128 x 128 fp32 tile and writes it back advanced by
//    accepted[b] tokens: 64 KB in and (when accepted > 0) 64 KB out per (sequence, value head);
//  * the layout the reference's engine hands its kernel (b200_gdn_verify_replay; qk_gdn_verify.cu:61-73,
//    586-593,631-647,706-717,769-781): a read-only fp32 checkpoint H0 per slot plus a 16-entry circular ring
//    of (d, k, g) per request, of which the first write_pos logical entries (physical entry
//    (cache_base + c) & 15) are committed.  The state the window sees is
//      S = e^{total} H0 + sum_c e^{total - pre_c} d_c k_c^T,   pre_c = g_0 + .. + g_c, total = pre_{wp-1},
//    so S x = e^{total} (H0 x) + sum_c e^{total - pre_c} d_c (k_c . x): the H0 products run on the tensor core,
//    the ring keys' dots against [q | k] on the CUDA cores.  Nothing is written to the checkpoint: the
//    window's D_s, unit keys and gates are appended to the ring as bf16 high and low parts (g in fp32) at
//    logical entries write_pos + s (those below 16), the conv state is rolled by the whole window and the
//    per-draft windows are recorded as [s1 s2 x0 x1 x2 x3] per channel; which of it survives is the engine's
//    move of the ring cursor.
//
// Two launches.  Only the state tile is bound by memory; everything else of a unit is a chain of dependent
// steps (input loads, conv, norms, barriers, dots, coefficients).  gdn_prep_kernel does all of that, once
// per (sequence, key head): conv + SiLU, norms, gates, window dots and coefficients, the conv-state roll (and,
// for the ring layout, the ring key dots, decay factors, ring appends and the window record), and leaves per
// key head one operand tile [q | k] already in the swizzled layout the tensor core reads plus, per value head,
// one 2.8 KB block (conv v, z, coefficients).  gdn_stream_kernel then only moves state tiles: per unit one TMA
// tensor load and two bulk copies, sixteen tf32 MMAs, the per-row epilogue, and for the explicit state the
// in-place update and the tile store.  It is launched with programmatic stream serialization and requests its
// first tile before waiting for the operand kernel, since the tile does not depend on it.
#include "common.cuh"
#include "host.h"

namespace b200 {

B200_DEFINE_WAIT_BUDGET_SETTER(set_wait_budget_gdn)

constexpr int G_HK = 16, G_HV = 32, G_D = 128, G_NT = 4;
constexpr int G_QDIM = G_HK * G_D;             // 2048
constexpr int G_CONV = 2 * G_QDIM + G_HV * G_D;  // 8192
constexpr int G_ZDIM = G_HV * G_D;             // 4096
constexpr int G_THREADS = 256;
constexpr int G_RING = 16;                     // ReplaySSM ring entries per request
constexpr uint32_t G_TILE_BYTES = G_D * G_D * 4;

__device__ __forceinline__ int sw_chunk(int row, int chunk) { return (chunk ^ (row & 7)) << 2; }  // float offset in a 32-float row

// One conv channel: window [s0 s1 s2 x0..x3] and the four taps, loaded up front so that every global
// load of the prologue is in flight at once.
struct ConvIn {
  bf16 win[G_NT + 3];
  uint2 w;
};
__device__ __forceinline__ void conv_load(const bf16* __restrict__ mixed_b, const bf16* __restrict__ cs_b,
                                          const bf16* __restrict__ conv_w, int ch, ConvIn& in) {
  in.win[0] = cs_b[ch * 3 + 0];
  in.win[1] = cs_b[ch * 3 + 1];
  in.win[2] = cs_b[ch * 3 + 2];
#pragma unroll
  for (int s = 0; s < G_NT; ++s) in.win[3 + s] = mixed_b[static_cast<size_t>(s) * G_CONV + ch];
  in.w = *reinterpret_cast<const uint2*>(conv_w + ch * 4);
}
// y[s] = bf16(silu(sum of bf16-rounded tap products, oldest first)) (conv_tap, qk_gdn_verify.cu:240-247)
__device__ __forceinline__ void conv_apply(const ConvIn& in, float (&y)[G_NT]) {
  const bf16 w0 = __ushort_as_bfloat16(in.w.x & 0xffff), w1 = __ushort_as_bfloat16(in.w.x >> 16);
  const bf16 w2 = __ushort_as_bfloat16(in.w.y & 0xffff), w3 = __ushort_as_bfloat16(in.w.y >> 16);
#pragma unroll
  for (int s = 0; s < G_NT; ++s) {
    float acc = bf2f(__hmul(in.win[s], w0));
    acc += bf2f(__hmul(in.win[s + 1], w1));
    acc += bf2f(__hmul(in.win[s + 2], w2));
    acc += bf2f(__hmul(in.win[s + 3], w3));
    y[s] = rbf(acc / (1.f + __expf(-acc)));
  }
}
// conv state after n_acc tokens = window elements [n_acc, n_acc + 3)
__device__ __forceinline__ void conv_roll(const ConvIn& in, bf16* __restrict__ cs_b, int ch, int n_acc) {
  if (n_acc <= 0) return;
  bf16 a = in.win[0], b = in.win[1], c = in.win[2];
#pragma unroll
  for (int n = 1; n <= G_NT; ++n)
    if (n_acc == n) {
      a = in.win[n];
      b = in.win[n + 1];
      c = in.win[n + 2];
    }
  cs_b[ch * 3 + 0] = a;
  cs_b[ch * 3 + 1] = b;
  cs_b[ch * 3 + 2] = c;
}

// the per-draft windows of a channel, deduplicated: [s1 s2 x0 x1 x2 x3] (Conv4::store, qk_gdn_verify.cu:277-289)
__device__ __forceinline__ void conv_record(const ConvIn& in, bf16* __restrict__ wrec, int ch) {
  uint32_t* dst = reinterpret_cast<uint32_t*>(wrec + static_cast<size_t>(ch) * 6);
#pragma unroll
  for (int i = 0; i < 3; ++i)
    dst[i] = static_cast<uint32_t>(__bfloat16_as_ushort(in.win[1 + 2 * i])) |
             (static_cast<uint32_t>(__bfloat16_as_ushort(in.win[2 + 2 * i])) << 16);
}

struct GdnArgs {
  const bf16* mixed;
  const bf16* z;
  const bf16* a;
  const bf16* b;
  bf16* conv_state;
  const bf16* conv_w;
  const float* a_log;
  const float* dt_bias;
  float* state;
  const int32_t* accepted;
  const bf16* norm_w;
  float eps;
  int B;
  bf16* out;
  int32_t* status;
  // REPLAY form: `state` is the read-only checkpoint pool, indexed by state_idx[b] like conv_state
  bf16* window;             // [window slots, 8192, 6]
  bf16* d_ring;             // [ring slots, 32, 16, 128] high parts (read and appended)
  bf16* dlo_ring;           // low parts (appended only)
  bf16* k_ring;             // [ring slots, 16, 16, 128]
  bf16* klo_ring;
  float* g_ring;            // [ring slots, 32, 16]
  const int32_t* state_idx;   // [B] checkpoint / conv-state slot, < 0: padded request (zero output, nothing written)
  const int32_t* ring_idx;    // [B] ring slot
  const int32_t* win_idx;     // [B] window slot
  const int32_t* write_pos;   // [ring slots] committed entries
  const int32_t* cache_base;  // [ring slots] physical entry of logical entry 0
};

// Optional timeline of the streaming kernel's CTA 0 (compile with -DB200_TRACE): %globaltimer stamps of thread 0 per
// unit at: 0 unit start, 1 tile and operands landed, 2 MMAs complete, 3 epilogue done, 4 outputs stored, 5 state
// updated and stores issued, 6 next unit requested; row 9: kernel start and end.
#ifdef B200_TRACE
__device__ unsigned long long g_gdn_trace[16][8];
#define G_TRACE(k, i) do { if (blockIdx.x == 0 && threadIdx.x == 0 && (i) < 8) g_gdn_trace[k][i] = globaltimer(); } while (0)
#else
#define G_TRACE(k, i) do { } while (0)
#endif

struct GdnOps {              // per (sequence, value head): one bulk copy
  bf16 v[G_NT][G_D];         // conv v (bf16 values)
  bf16 z[G_NT][G_D];         // gate input
  float cA[G_NT][G_NT], cF[G_NT][G_NT], cE[G_NT], cR[G_NT], cC[G_NT];
  int n_acc;                 // explicit state: tokens to advance the state by
  int skip;                  // ring layout: padded request, nothing to do
  int ring, wp, cb;          // ring layout: ring slot, committed entries (0..16), physical entry of logical entry 0
  float tdec;                // ring layout: e^{total}
  int pad[2];
  float dec[G_RING];         // ring layout: e^{total - pre_c}, 0 past the history
  float xr[G_RING][8];       // ring layout: ring key c . [q | k], 0 past the history
};
static_assert(sizeof(GdnOps) == 2832 && sizeof(GdnOps) % 16 == 0, "GdnOps is copied with one bulk copy");
constexpr int G_QK_FLOATS = 4 * 8 * 32;  // the operand tile of one (sequence, key head): 4 KB

struct GdnPrepSmem {
  float q[G_NT][G_D], k[G_NT][G_D];
  float nrm[2][G_NT][4];
  float kk[G_NT][G_NT], kq[G_NT][G_NT];
  float g[2][G_NT], beta[2][G_NT];
  float xr[G_RING][8];
  float gr[2][G_RING];
};

template <bool REPLAY>
__global__ void __launch_bounds__(512, 4) gdn_prep_kernel(const GdnArgs p, float* __restrict__ qk_ws, GdnOps* __restrict__ ops_ws) {
  __shared__ GdnPrepSmem sm;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int pair = blockIdx.x, b = pair / G_HK, hk = pair - b * G_HK;
  const int grp = tid >> 7, c = tid & 127;  // 0: q, 1: k, 2 / 3: v of value head 2 hk / 2 hk + 1
  pdl_wait();
  pdl_launch();
  int slot = b, ring = 0, wslot = 0, wp = 0, cb = 0, n_acc = G_NT;
  if constexpr (REPLAY) {
    slot = p.state_idx[b];
    if (slot < 0) {  // padded request: zero rows, and the streaming kernel is told to skip both units
      if (grp >= 2) {
        const int hv = 2 * hk + grp - 2;
#pragma unroll
        for (int s = 0; s < G_NT; ++s) p.out[(static_cast<size_t>(b) * G_NT + s) * G_ZDIM + hv * G_D + c] = f2bf(0.f);
        if (c == 0) ops_ws[b * G_HV + hv].skip = 1;
      }
      return;
    }
    ring = p.ring_idx[b];
    wslot = p.win_idx[b];
    wp = p.write_pos[ring];
    cb = p.cache_base[ring];
    wp = wp < 0 ? 0 : (wp > G_RING ? G_RING : wp);
  } else {
    n_acc = p.accepted[b];
    n_acc = n_acc < 0 ? 0 : (n_acc > G_NT ? G_NT : n_acc);
  }
  const bf16* mixed_b = p.mixed + static_cast<size_t>(b) * G_NT * G_CONV;
  bf16* cs_b = p.conv_state + static_cast<size_t>(slot) * G_CONV * 3;
  const int hv_mine = 2 * hk + (grp & 1);  // value head of a v thread
  const int ch = grp == 0 ? hk * G_D + c : (grp == 1 ? G_QDIM + hk * G_D + c : 2 * G_QDIM + hv_mine * G_D + c);
  ConvIn in;
  conv_load(mixed_b, cs_b, p.conv_w, ch, in);
  bf16 zraw[G_NT];
  if (grp >= 2) {
#pragma unroll
    for (int s = 0; s < G_NT; ++s) zraw[s] = p.z[(static_cast<size_t>(b) * G_NT + s) * G_ZDIM + hv_mine * G_D + c];
  }
  if (tid < 2 * G_NT) {  // gates of both value heads (qk_gdn_verify.cu:616-631)
    const int h = tid >> 2, s = tid & 3, hv = 2 * hk + h;
    const float av = bf2f(p.a[(static_cast<size_t>(b) * G_NT + s) * G_HV + hv]);
    const float bv = bf2f(p.b[(static_cast<size_t>(b) * G_NT + s) * G_HV + hv]);
    const float xg = av + p.dt_bias[hv];
    const float sp = xg <= 20.f ? log1pf(expf(xg)) : xg;
    const float g = -expf(p.a_log[hv]) * sp;
    sm.g[h][s] = g;
    sm.beta[h][s] = 1.f / (1.f + expf(-bv));
    if constexpr (REPLAY)
      if (wp + s < G_RING) p.g_ring[(static_cast<size_t>(ring) * G_HV + hv) * G_RING + ((cb + wp + s) & (G_RING - 1))] = g;
  } else if (REPLAY && tid >= 32 && tid < 64) {
    const int h = (tid - 32) >> 4, e = tid & 15;
    sm.gr[h][e] = e < wp ? p.g_ring[(static_cast<size_t>(ring) * G_HV + 2 * hk + h) * G_RING + ((cb + e) & (G_RING - 1))] : 0.f;
  }
  uint2 rk = make_uint2(0u, 0u);  // ring layout: warp w multiplies committed key w
  if constexpr (REPLAY)
    if (warp < wp)
      rk = *reinterpret_cast<const uint2*>(p.k_ring + ((static_cast<size_t>(ring) * G_HK + hk) * G_RING +
                                                       ((cb + warp) & (G_RING - 1))) * G_D + 4 * lane);
  float y[G_NT];
  conv_apply(in, y);
  if (grp < 2) {
    float ss[G_NT];
#pragma unroll
    for (int s = 0; s < G_NT; ++s) ss[s] = y[s] * y[s];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1)
#pragma unroll
      for (int s = 0; s < G_NT; ++s) ss[s] += __shfl_xor_sync(FULL_MASK, ss[s], o);
    if (lane == 0)
#pragma unroll
      for (int s = 0; s < G_NT; ++s) sm.nrm[grp][s][warp & 3] = ss[s];
  } else {
    GdnOps& o = ops_ws[b * G_HV + hv_mine];
#pragma unroll
    for (int s = 0; s < G_NT; ++s) {
      o.v[s][c] = f2bf(y[s]);
      o.z[s][c] = zraw[s];
    }
  }
  // every channel belongs to this CTA alone, and its old conv state is in registers: roll it
  conv_roll(in, cs_b, ch, n_acc);
  if constexpr (REPLAY) conv_record(in, p.window + static_cast<size_t>(wslot) * G_CONV * 6, ch);
  __syncthreads();
  if (grp < 2) {
    const int sub = c >> 5, chk = (c & 31) >> 2, e = c & 3;
    float* qk = qk_ws + static_cast<size_t>(pair) * G_QK_FLOATS;
#pragma unroll
    for (int s = 0; s < G_NT; ++s) {
      const float n = sm.nrm[grp][s][0] + sm.nrm[grp][s][1] + sm.nrm[grp][s][2] + sm.nrm[grp][s][3];
      const float r = (1.f / sqrtf(n + 1e-6f)) * (grp ? 1.f : 0.08838834764831845f);  // d_k^-0.5 on q
      const float val = y[s] * r;
      const int row = grp * 4 + s;
      qk[sub * 256 + row * 32 + sw_chunk(row, chk) + e] = val;
      (grp ? sm.k : sm.q)[s][c] = val;
      if constexpr (REPLAY) {
        if (grp == 1 && wp + s < G_RING) {  // unit keys join the ring as high and low parts (qk_gdn_verify.cu:586-593)
          const size_t at = ((static_cast<size_t>(ring) * G_HK + hk) * G_RING + ((cb + wp + s) & (G_RING - 1))) * G_D + c;
          const bf16 hi = f2bf(val);
          p.k_ring[at] = hi;
          p.klo_ring[at] = f2bf(val - bf2f(hi));
        }
      }
    }
  }
  __syncthreads();
  // k_i . k_j and k_i . q_j: 32 dots of length 128, two per warp
#pragma unroll
  for (int dd = 0; dd < 2; ++dd) {
    const int d = 2 * warp + dd, i = (d >> 2) & 3, j = d & 3;
    float acc = 0.f;
#pragma unroll
    for (int c4 = 0; c4 < 4; ++c4) {
      const int cc = lane + 32 * c4;
      acc = fmaf(sm.k[i][cc], d < 16 ? sm.k[j][cc] : sm.q[j][cc], acc);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(FULL_MASK, acc, o);
    if (lane == 0) (d < 16 ? sm.kk : sm.kq)[i][j] = acc;
  }
  if constexpr (REPLAY) {
    // committed ring key `warp` against [q | k] (qk_gdn_verify.cu:597-604,662-671); columns summed over the lanes
    // by a transposing butterfly (lane l ends with column (l >> 4 & 1) * 4 + (l >> 3 & 1) * 2 + (l >> 2 & 1))
    if (warp < wp) {
      const float k0 = bf_lo(rk.x), k1 = bf_hi(rk.x), k2 = bf_lo(rk.y), k3 = bf_hi(rk.y);
      float acc[8];
#pragma unroll
      for (int s = 0; s < G_NT; ++s) {
        const float4 cq = *reinterpret_cast<const float4*>(&sm.q[s][4 * lane]);
        const float4 ck = *reinterpret_cast<const float4*>(&sm.k[s][4 * lane]);
        acc[s] = fmaf(k3, cq.w, fmaf(k2, cq.z, fmaf(k1, cq.y, k0 * cq.x)));
        acc[4 + s] = fmaf(k3, ck.w, fmaf(k2, ck.z, fmaf(k1, ck.y, k0 * ck.x)));
      }
      float a4[4], a2[2], a1;
      {
        const bool up = lane & 16;
#pragma unroll
        for (int n = 0; n < 4; ++n) {
          const float give = up ? acc[n] : acc[4 + n], keep = up ? acc[4 + n] : acc[n];
          a4[n] = keep + __shfl_xor_sync(FULL_MASK, give, 16);
        }
      }
      {
        const bool up = lane & 8;
#pragma unroll
        for (int n = 0; n < 2; ++n) {
          const float give = up ? a4[n] : a4[2 + n], keep = up ? a4[2 + n] : a4[n];
          a2[n] = keep + __shfl_xor_sync(FULL_MASK, give, 8);
        }
      }
      {
        const bool up = lane & 4;
        const float give = up ? a2[0] : a2[1], keep = up ? a2[1] : a2[0];
        a1 = keep + __shfl_xor_sync(FULL_MASK, give, 4);
      }
      a1 += __shfl_xor_sync(FULL_MASK, a1, 2);
      a1 += __shfl_xor_sync(FULL_MASK, a1, 1);
      if ((lane & 3) == 0) sm.xr[warp][((lane >> 4) & 1) * 4 + ((lane >> 3) & 1) * 2 + ((lane >> 2) & 1)] = a1;
    } else if (lane < 8) {
      sm.xr[warp][lane] = 0.f;
    }
  }
  __syncthreads();
  if (warp < 2) {
    // the window's scalar coefficients of value head 2 hk + warp
    GdnOps& o = ops_ws[b * G_HV + 2 * hk + warp];
    float G[G_NT];
    float run = 0.f;
#pragma unroll
    for (int s = 0; s < G_NT; ++s) {
      run += sm.g[warp][s];
      G[s] = run;
    }
    if (lane < 16) {
      const int i = lane >> 2, j = lane & 3;
      float Gi = 0.f, Gj = 0.f;
#pragma unroll
      for (int s = 0; s < G_NT; ++s) {
        Gi = s == i ? G[s] : Gi;
        Gj = s == j ? G[s] : Gj;
      }
      o.cA[i][j] = i > j ? sm.beta[warp][i] * __expf(Gi - Gj) * sm.kk[i][j] : 0.f;
      o.cF[i][j] = i <= j ? __expf(Gj - Gi) * sm.kq[i][j] : 0.f;
    } else if (lane < 20) {
      const int s = lane - 16;
      float Gs = 0.f, Gn = 0.f;
#pragma unroll
      for (int u = 0; u < G_NT; ++u) {
        Gs = u == s ? G[u] : Gs;
        Gn = u == n_acc - 1 ? G[u] : Gn;
      }
      o.cE[s] = __expf(Gs);
      o.cR[s] = sm.beta[warp][s];
      o.cC[s] = s < n_acc ? __expf(Gn - Gs) : 0.f;
    } else if (lane == 20) {
      o.n_acc = n_acc;
      o.skip = 0;
      o.ring = ring;
      o.wp = wp;
      o.cb = cb;
      if constexpr (!REPLAY) o.tdec = 1.f;
    }
  } else if (REPLAY && warp < 4) {
    // decay of every committed entry up to the window and of the checkpoint (qk_gdn_verify.cu:633-647)
    GdnOps& o = ops_ws[b * G_HV + 2 * hk + warp - 2];
    const int e = lane & 15;
    float pre = sm.gr[warp - 2][e];
#pragma unroll
    for (int off = 1; off < G_RING; off <<= 1) {
      const float n = __shfl_up_sync(FULL_MASK, pre, off, G_RING);
      if (e >= off) pre += n;
    }
    const float total = __shfl_sync(FULL_MASK, pre, G_RING - 1, G_RING);
    if (lane < G_RING) {
      o.dec[e] = e < wp ? __expf(total - pre) : 0.f;
      if (e == 0) o.tdec = __expf(total);
    }
  } else if (REPLAY && tid >= 128 && tid < 384) {
    const int idx = tid - 128, h = idx >> 7, j = idx & 127;
    ops_ws[b * G_HV + 2 * hk + h].xr[j >> 3][j & 7] = sm.xr[j >> 3][j & 7];
  }
}

struct GdnStreamSmem {
  float S[4][G_D * 32];   // 64 KB state tile, swizzled sub-tiles (1024-byte aligned)
  float QK[4][8 * 32];    // operand tile [q | k]; the MMA's rows 8..15 alias what follows.  Ring layout: once the
                          // MMAs are done, the value head's 16 d entries (bf16 [physical entry][value row])
  GdnOps ops;             // explicit state: v and z are overwritten by c_i D_i (fp32 [4][128]) for the state update
  float red[4][G_NT];
  uint64_t bar_tile, bar_ops, bar_mma, bar_d;
  uint32_t tmem_slot;
  int abort_flag;
};

// Persistent CTAs, three per SM; unit u = (sequence, value head) = blockIdx.x + i * gridDim.x.
// REPLAY (checkpoint + ring layout): the tile is only read, so the next unit's tile is requested as soon as this
// unit's MMAs have left the buffer; the d entries are copied over the consumed operand tile; padded requests
// (ops.skip) use no tile.
template <bool REPLAY>
__global__ void __launch_bounds__(G_THREADS, 3)
gdn_stream_kernel(const __grid_constant__ CUtensorMap tmS, const GdnArgs p, const float* __restrict__ qk_ws,
                  const GdnOps* __restrict__ ops_ws) {
  extern __shared__ uint8_t smem_raw[];
  GdnStreamSmem& sm = *reinterpret_cast<GdnStreamSmem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int nunits = p.B * G_HV;
  if (tid == 0) {
    mbar_init(&sm.bar_tile, 1);
    mbar_init(&sm.bar_ops, 1);
    mbar_init(&sm.bar_mma, 1);
    mbar_init(&sm.bar_d, 1);
    sm.abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmS);
  }
  if (warp == 0) tmem_alloc(&sm.tmem_slot, 32);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = sm.tmem_slot;
  G_TRACE(9, 0);
  int unit_no = 0;
  // thread 0 keeps the phases it has armed and not yet seen complete (-1: none), for the wind-down after an
  // abandoned wait
  int pend_tile = -1, pend_ops = -1, pend_d = -1;
  uint32_t par_t = 0, par_o = 0, par_d = 0;  // phases of bar_tile (and bar_mma), bar_ops, bar_d of the current unit
  auto request_tile = [&](int u, int slot, uint32_t phase) {  // first state row of the unit: (slot * 32 + head) * 128
    mbar_expect_tx(&sm.bar_tile, G_TILE_BYTES);
#pragma unroll
    for (int sub = 0; sub < 4; ++sub) tma_load_2d(sm.S[sub], &tmS, 32 * sub, (slot * G_HV + (u & 31)) * G_D, &sm.bar_tile);
    pend_tile = static_cast<int>(phase);
  };
  auto request_ops = [&](int u, uint32_t phase) {
    mbar_expect_tx(&sm.bar_ops, G_QK_FLOATS * 4 + sizeof(GdnOps));
    bulk_load(sm.QK, qk_ws + static_cast<size_t>(u >> 1) * G_QK_FLOATS, G_QK_FLOATS * 4, &sm.bar_ops);
    bulk_load(&sm.ops, ops_ws + u, sizeof(GdnOps), &sm.bar_ops);
    pend_ops = static_cast<int>(phase);
  };
  // the first tile does not depend on the operand kernel: it travels while that kernel runs
  int nslot = -1;  // thread 0: state slot of the unit whose tile is requested next
  if (tid == 0 && blockIdx.x < nunits) {
    nslot = REPLAY ? p.state_idx[blockIdx.x >> 5] : static_cast<int>(blockIdx.x >> 5);
    if (nslot >= 0) request_tile(blockIdx.x, nslot, 0);
  }
  pdl_wait();
  if (tid == 0 && blockIdx.x < nunits) request_ops(blockIdx.x, 0);
  bool ok = true;
  for (int u = blockIdx.x; u < nunits; u += gridDim.x, par_o ^= 1u) {
    const int b = u >> 5, hv = u & 31;
    const int un = u + gridDim.x;  // this CTA's next unit
    G_TRACE(0, unit_no);
    if (tid == 0) nslot = un < nunits ? (REPLAY ? p.state_idx[un >> 5] : (un >> 5)) : -1;  // consumed much later
    if constexpr (REPLAY) {
      ok = mbar_wait(&sm.bar_ops, par_o, &sm.abort_flag, p.status, ST_WAIT_FULL);
      ok = __syncthreads_and(ok);
      if (!ok) break;
      if (tid == 0) pend_ops = -1;
      if (sm.ops.skip) {  // padded request: the operand kernel has zeroed its rows; no tile was requested
        __syncthreads();  // every thread has read the flag
        if (tid == 0 && un < nunits) {
          request_ops(un, par_o ^ 1u);
          if (nslot >= 0) request_tile(un, nslot, par_t);
        }
        continue;
      }
    }
    // ---- S [q | k]: sixteen tf32 MMAs (M = 128 state rows, N = 16, K = 8 each) into 16 TMEM columns ----
    if (tid == 0) {
      const bool landed = mbar_wait(&sm.bar_tile, par_t, &sm.abort_flag, p.status, ST_WAIT_STATE) &&
                          mbar_wait(&sm.bar_ops, par_o, &sm.abort_flag, p.status, ST_WAIT_FULL);
      G_TRACE(1, unit_no);
      if (landed) {
        pend_tile = pend_ops = -1;
        tc_fence_after();
        const uint32_t idesc = umma_idesc(UMMA_C_F32, UMMA_AB_TF32, 16);
#pragma unroll
        for (int sub = 0; sub < 4; ++sub)
#pragma unroll
          for (int kk = 0; kk < 4; ++kk)
            tc_mma_tf32(tmem_base, umma_desc_sw128(smem_u32(sm.S[sub]) + kk * 32),
                        umma_desc_sw128(smem_u32(sm.QK[sub]) + kk * 32), idesc, (sub | kk) != 0);
        tc_commit(&sm.bar_mma);
      }
    }
    ok = mbar_wait(&sm.bar_ops, par_o, &sm.abort_flag, p.status, ST_WAIT_FULL) &&
         mbar_wait(&sm.bar_tile, par_t, &sm.abort_flag, p.status, ST_WAIT_STATE) &&
         mbar_wait(&sm.bar_mma, par_t, &sm.abort_flag, p.status, ST_WAIT_TMEM_FULL);
    ok = __syncthreads_and(ok);  // one verdict for the CTA
    if (!ok) break;
    tc_fence_after();
    G_TRACE(2, unit_no);
    const int n_acc = sm.ops.n_acc;
    if constexpr (REPLAY) {
      // the MMAs were the only readers of the tile and of the operand tile: the d entries of the value head (4 KB,
      // physical order) land on the operand tile, and the next unit's checkpoint tile may travel
      if (tid == 0) {
        mbar_expect_tx(&sm.bar_d, G_RING * G_D * 2);
        bulk_load(sm.QK, p.d_ring + (static_cast<size_t>(sm.ops.ring) * G_HV + hv) * G_RING * G_D, G_RING * G_D * 2, &sm.bar_d);
        pend_d = static_cast<int>(par_d);
        if (nslot >= 0) request_tile(un, nslot, par_t ^ 1u);
      }
      ok = mbar_wait(&sm.bar_d, par_d, &sm.abort_flag, p.status, ST_WAIT_FULL);
      ok = __syncthreads_and(ok);
      if (!ok) break;
      if (tid == 0) pend_d = -1;
    }
    // ---- per value row: R, D = (I + A)^-1 R, outputs; gated RMSNorm ----
    float o[G_NT] = {0.f, 0.f, 0.f, 0.f}, zz[G_NT] = {0.f, 0.f, 0.f, 0.f}, cd[G_NT] = {0.f, 0.f, 0.f, 0.f};
    if (tid < G_D) {
      const int v = tid;
      uint32_t hr[16];
      tmem_ld16(tmem_base + (static_cast<uint32_t>(warp * 32) << 16), hr);  // warps 0..3 own TMEM lane quadrants 0..3
      tmem_ld_wait();
      float hq[G_NT], hk_[G_NT];
#pragma unroll
      for (int s = 0; s < G_NT; ++s) {
        hq[s] = __uint_as_float(hr[s]);
        hk_[s] = __uint_as_float(hr[4 + s]);
      }
      if constexpr (REPLAY) {
        // S x = e^{total} H0 x + sum_c (d_c e^{total - pre_c}) (k_c . x)   (qk_gdn_verify.cu:706-742)
        const bf16* dsm = reinterpret_cast<const bf16*>(&sm.QK[0][0]);
        const int wp = sm.ops.wp, cb = sm.ops.cb;
        float aq[G_NT] = {0.f, 0.f, 0.f, 0.f}, ak[G_NT] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll 4
        for (int e = 0; e < wp; ++e) {
          const float dsc = bf2f(dsm[((cb + e) & (G_RING - 1)) * G_D + v]) * sm.ops.dec[e];
          const float4 xq = *reinterpret_cast<const float4*>(&sm.ops.xr[e][0]);
          const float4 xk = *reinterpret_cast<const float4*>(&sm.ops.xr[e][4]);
          aq[0] = fmaf(dsc, xq.x, aq[0]); aq[1] = fmaf(dsc, xq.y, aq[1]);
          aq[2] = fmaf(dsc, xq.z, aq[2]); aq[3] = fmaf(dsc, xq.w, aq[3]);
          ak[0] = fmaf(dsc, xk.x, ak[0]); ak[1] = fmaf(dsc, xk.y, ak[1]);
          ak[2] = fmaf(dsc, xk.z, ak[2]); ak[3] = fmaf(dsc, xk.w, ak[3]);
        }
        const float td = sm.ops.tdec;
#pragma unroll
        for (int s = 0; s < G_NT; ++s) {
          hq[s] = fmaf(td, hq[s], aq[s]);
          hk_[s] = fmaf(td, hk_[s], ak[s]);
        }
      }
      float R[G_NT], D[G_NT];
#pragma unroll
      for (int s = 0; s < G_NT; ++s) {
        zz[s] = bf2f(sm.ops.z[s][v]);
        R[s] = sm.ops.cR[s] * (bf2f(sm.ops.v[s][v]) - sm.ops.cE[s] * hk_[s]);
      }
#pragma unroll
      for (int i = 0; i < G_NT; ++i) {
        float d = R[i];
#pragma unroll
        for (int j = 0; j < i; ++j) d = fmaf(-sm.ops.cA[i][j], D[j], d);
        D[i] = d;
      }
#pragma unroll
      for (int s = 0; s < G_NT; ++s) {
        float acc = sm.ops.cE[s] * hq[s];
#pragma unroll
        for (int i = 0; i <= s; ++i) acc = fmaf(D[i], sm.ops.cF[i][s], acc);
        o[s] = rbf(acc);  // the core output is stored in bf16 before the norm (qk_gdn_verify.cu:761)
        cd[s] = D[s] * sm.ops.cC[s];
      }
      if constexpr (REPLAY) {
        // the window's D join the ring as bf16 high and low parts (qk_gdn_verify.cu:769-781)
        const int wp = sm.ops.wp, cb = sm.ops.cb;
        const size_t base = (static_cast<size_t>(sm.ops.ring) * G_HV + hv) * G_RING * G_D + v;
#pragma unroll
        for (int s = 0; s < G_NT; ++s)
          if (wp + s < G_RING) {
            const size_t at = base + static_cast<size_t>((cb + wp + s) & (G_RING - 1)) * G_D;
            const bf16 hi = f2bf(D[s]);
            p.d_ring[at] = hi;
            p.dlo_ring[at] = f2bf(D[s] - bf2f(hi));
          }
      }
      float ss[G_NT];
#pragma unroll
      for (int s = 0; s < G_NT; ++s) ss[s] = o[s] * o[s];
#pragma unroll
      for (int off = 16; off > 0; off >>= 1)
#pragma unroll
        for (int s = 0; s < G_NT; ++s) ss[s] += __shfl_xor_sync(FULL_MASK, ss[s], off);
      if (lane == 0)
#pragma unroll
        for (int s = 0; s < G_NT; ++s) sm.red[warp][s] = ss[s];
    }
    tc_fence_before();
    G_TRACE(3, unit_no);
    __syncthreads();  // row sums visible; every thread has read its v and z
    float* cdsm = reinterpret_cast<float*>(&sm.ops.v[0][0]);  // c_i D_i, fp32 [4][128], over v and z
    if (tid < G_D) {
      const float nw = bf2f(p.norm_w[tid]);
#pragma unroll
      for (int s = 0; s < G_NT; ++s) {
        const float var = (sm.red[0][s] + sm.red[1][s] + sm.red[2][s] + sm.red[3][s]) * (1.f / G_D);
        const float rstd = rsqrtf(var + p.eps);
        p.out[(static_cast<size_t>(b) * G_NT + s) * G_ZDIM + hv * G_D + tid] =
            f2bf(o[s] * rstd * nw * (zz[s] * (1.f / (1.f + __expf(-zz[s])))));
        if constexpr (!REPLAY) cdsm[s * G_D + tid] = cd[s];
      }
    }
    G_TRACE(4, unit_no);
    // ---- state after n_acc tokens, in place in the swizzled tile, then four TMA tensor stores ----
    if (!REPLAY && n_acc > 0) {
      __syncthreads();  // c_i D_i visible
      const int rg = tid >> 3, ks = tid & 7;  // thread = 4 state rows x one 16-byte chunk position of each sub-tile row
      const float decay = sm.ops.cE[n_acc - 1];
      float cdr[4][G_NT];
#pragma unroll
      for (int r = 0; r < 4; ++r)
#pragma unroll
        for (int i = 0; i < G_NT; ++i) cdr[r][i] = cdsm[i * G_D + rg * 4 + r];
#pragma unroll
      for (int sub = 0; sub < 4; ++sub) {
        float4 kv[G_NT];
#pragma unroll
        for (int t = 0; t < G_NT; ++t) kv[t] = *reinterpret_cast<const float4*>(&sm.QK[sub][(4 + t) * 32 + sw_chunk(4 + t, ks)]);
#pragma unroll
        for (int r = 0; r < 4; ++r) {
          const int row = rg * 4 + r;
          float4* sp = reinterpret_cast<float4*>(&sm.S[sub][row * 32 + sw_chunk(row, ks)]);
          float4 sv = *sp;
          sv.x *= decay; sv.y *= decay; sv.z *= decay; sv.w *= decay;
#pragma unroll
          for (int t = 0; t < G_NT; ++t) {
            sv.x = fmaf(cdr[r][t], kv[t].x, sv.x);
            sv.y = fmaf(cdr[r][t], kv[t].y, sv.y);
            sv.z = fmaf(cdr[r][t], kv[t].z, sv.z);
            sv.w = fmaf(cdr[r][t], kv[t].w, sv.w);
          }
          *sp = sv;
        }
        // this 16 KB sub-tile is final: hand it to TMA while the next one is being updated
        fence_proxy_async();
        __syncthreads();
        if (tid == 0) {
          tma_store_2d(&tmS, 32 * sub, u * G_D, sm.S[sub]);
          bulk_commit();
        }
      }
      G_TRACE(5, unit_no);
      // the operand blocks are free: the next unit's may travel while the tile leaves
      if (tid == 0 && un < nunits) {
        request_ops(un, par_o ^ 1u);
        bulk_wait_read_all();  // the tile has left shared memory
        request_tile(un, nslot, par_t ^ 1u);
      }
      G_TRACE(6, unit_no);
    } else {
      __syncthreads();  // every thread is done with the operand blocks (and, explicit state, with the tile)
      if (tid == 0 && un < nunits) {
        request_ops(un, par_o ^ 1u);
        if constexpr (!REPLAY) request_tile(un, nslot, par_t ^ 1u);
      }
    }
    par_t ^= 1u;
    par_d ^= 1u;
    ++unit_no;
  }
  G_TRACE(9, 1);
  if (!ok && tid == 0) {
    // an abandoned wait: give the copies in flight a bounded grace period before the CTA's memory goes away
    const unsigned long long t0 = globaltimer();
    while (globaltimer() - t0 < 20000000ull) {
      if (pend_tile >= 0 && mbar_try(&sm.bar_tile, static_cast<uint32_t>(pend_tile))) pend_tile = -1;
      if (pend_ops >= 0 && mbar_try(&sm.bar_ops, static_cast<uint32_t>(pend_ops))) pend_ops = -1;
      if (pend_d >= 0 && mbar_try(&sm.bar_d, static_cast<uint32_t>(pend_d))) pend_d = -1;
      if (pend_tile < 0 && pend_ops < 0 && pend_d < 0) break;
    }
  }
  if (tid == 0) bulk_wait_read_all();  // the last tile has left shared memory; the writes complete with the grid
  __syncthreads();
  if (warp == 0) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 32);
  }
}


// Fold of the committed ring entries into the checkpoint (the step the reference leaves to its engine's pool,
// gdn_fused.py:24 `replayssm_spec_fold`): H0 <- e^{total} H0 + sum_{c < wp} e^{total - pre_c} d_c k_c^T with the full
// entries (high + low parts).  One CTA per (request, value head); thread = one 16-byte column group of 16 rows, so
// every access to the tile is a coalesced 512-byte row.  The cursors stay the caller's: after the fold it sets
// write_pos to 0.
struct GdnFoldArgs {
  float* checkpoint;
  const bf16 *d_ring, *dlo_ring, *k_ring, *klo_ring;
  const float* g_ring;
  const int32_t *state_idx, *ring_idx, *write_pos, *cache_base;
};

__global__ void __launch_bounds__(256) gdn_fold_kernel(const GdnFoldArgs p) {
  __shared__ float dco[G_RING][G_D];  // e^{total - pre_c} d_c[v]
  __shared__ float ks[G_RING][G_D];   // k_c
  __shared__ float dec[G_RING];
  __shared__ float tdec;
  const int tid = threadIdx.x, b = blockIdx.x / G_HV, hv = blockIdx.x % G_HV;
  pdl_wait();
  pdl_launch();
  const int slot = p.state_idx[b];
  if (slot < 0) return;
  const int ring = p.ring_idx[b], cb = p.cache_base[ring];
  int wp = p.write_pos[ring];
  wp = wp < 0 ? 0 : (wp > G_RING ? G_RING : wp);
  if (wp == 0) return;  // nothing committed: the checkpoint is the state
  if (tid < 32) {
    const int e = tid & 15;
    float pre = e < wp ? p.g_ring[(static_cast<size_t>(ring) * G_HV + hv) * G_RING + ((cb + e) & (G_RING - 1))] : 0.f;
#pragma unroll
    for (int o = 1; o < G_RING; o <<= 1) {
      const float n = __shfl_up_sync(FULL_MASK, pre, o, G_RING);
      if (e >= o) pre += n;
    }
    const float total = __shfl_sync(FULL_MASK, pre, G_RING - 1, G_RING);
    if (tid < G_RING) {
      dec[e] = e < wp ? expf(total - pre) : 0.f;
      if (e == 0) tdec = expf(total);
    }
  }
  __syncthreads();
  for (int i = tid; i < wp * G_D; i += 256) {
    const int e = i >> 7, c = i & 127, ph = (cb + e) & (G_RING - 1);
    const size_t dat = ((static_cast<size_t>(ring) * G_HV + hv) * G_RING + ph) * G_D + c;
    const size_t kat = ((static_cast<size_t>(ring) * G_HK + (hv >> 1)) * G_RING + ph) * G_D + c;
    dco[e][c] = (bf2f(p.d_ring[dat]) + bf2f(p.dlo_ring[dat])) * dec[e];
    ks[e][c] = bf2f(p.k_ring[kat]) + bf2f(p.klo_ring[kat]);
  }
  __syncthreads();
  float* tile = p.checkpoint + (static_cast<size_t>(slot) * G_HV + hv) * G_D * G_D;
  const int col = (tid & 31) * 4, r0 = tid >> 5;
  const float td = tdec;
  float4 acc[16];
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    acc[i] = *reinterpret_cast<const float4*>(tile + (r0 + 8 * i) * G_D + col);
    acc[i].x *= td; acc[i].y *= td; acc[i].z *= td; acc[i].w *= td;
  }
  for (int e = 0; e < wp; ++e) {
    const float4 kv = *reinterpret_cast<const float4*>(&ks[e][col]);
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const float d = dco[e][r0 + 8 * i];
      acc[i].x = fmaf(d, kv.x, acc[i].x);
      acc[i].y = fmaf(d, kv.y, acc[i].y);
      acc[i].z = fmaf(d, kv.z, acc[i].z);
      acc[i].w = fmaf(d, kv.w, acc[i].w);
    }
  }
#pragma unroll
  for (int i = 0; i < 16; ++i) *reinterpret_cast<float4*>(tile + (r0 + 8 * i) * G_D + col) = acc[i];
}

}  // namespace b200

using namespace b200;

#ifdef B200_TRACE
extern "C" int b200_gdn_trace_read(unsigned long long* host) {
  return static_cast<int>(cudaMemcpyFromSymbol(host, g_gdn_trace, sizeof(g_gdn_trace)));
}
#endif

extern "C" size_t b200_gdn_workspace_bytes(int B) {
  return B <= 0 ? 0 : static_cast<size_t>(B) * (G_HK * G_QK_FLOATS * 4 + G_HV * sizeof(GdnOps));
}

// operand kernel, then streaming kernel (three CTAs per SM by shared memory), both with programmatic stream
// serialization
template <bool REPLAY>
static int gdn_launch(const CUtensorMap& tmS, const GdnArgs& p, int B, void* ws, size_t ws_bytes, void* stream,
                      const char* what) {
  if (!ws || ws_bytes < b200_gdn_workspace_bytes(B))
    return fail(B200_E_WS, "%s: workspace of %zu bytes needed, %zu given", what, b200_gdn_workspace_bytes(B), ws_bytes);
  if (reinterpret_cast<uintptr_t>(ws) & 127) return fail(B200_E_ALIGN, "%s: workspace must be 128-byte aligned", what);
  float* qk_ws = static_cast<float*>(ws);
  GdnOps* ops_ws = reinterpret_cast<GdnOps*>(qk_ws + static_cast<size_t>(B) * G_HK * G_QK_FLOATS);
  const int smem = static_cast<int>(sizeof(GdnStreamSmem)) + 1024;
  static DeviceOnce once;  // one per instantiation of this function template
  once.run([smem] { cudaFuncSetAttribute(gdn_stream_kernel<REPLAY>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem); });
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  launch_k(gdn_prep_kernel<REPLAY>, dim3(B * G_HK), dim3(512), 0, st, p, qk_ws, ops_ws);
  int grid = sm_count() * 3;
  if (grid > B * G_HV) grid = B * G_HV;
  launch_k(gdn_stream_kernel<REPLAY>, dim3(grid), dim3(G_THREADS), static_cast<size_t>(smem), st, tmS, p,
           static_cast<const float*>(qk_ws), static_cast<const GdnOps*>(ops_ws));
  return launch_status(what);
}

extern "C" int b200_gdn_verify(const void* mixed, const void* z, const void* a, const void* b, void* conv_state,
                               const void* conv_w, const float* a_log, const float* dt_bias, float* state,
                               const int32_t* accepted, const void* norm_w, float eps, int B, void* out, void* ws,
                               size_t ws_bytes, int32_t* status, void* stream) {
  if (!mixed || !z || !a || !b || !conv_state || !conv_w || !a_log || !dt_bias || !state || !accepted || !norm_w || !out)
    return fail(B200_E_ARG, "b200_gdn_verify: null pointer");
  if (B < 0 || B > 65535) return fail(B200_E_ARG, "b200_gdn_verify: B=%d out of range", B);
  if (reinterpret_cast<uintptr_t>(state) & 15) return fail(B200_E_ALIGN, "b200_gdn_verify: state must be 16-byte aligned");
  if (reinterpret_cast<uintptr_t>(conv_w) & 7) return fail(B200_E_ALIGN, "b200_gdn_verify: conv_w must be 8-byte aligned");
  if (B == 0) return 0;
  GdnArgs p{};
  p.mixed = static_cast<const bf16*>(mixed);
  p.z = static_cast<const bf16*>(z);
  p.a = static_cast<const bf16*>(a);
  p.b = static_cast<const bf16*>(b);
  p.conv_state = static_cast<bf16*>(conv_state);
  p.conv_w = static_cast<const bf16*>(conv_w);
  p.a_log = a_log;
  p.dt_bias = dt_bias;
  p.state = state;
  p.accepted = accepted;
  p.norm_w = static_cast<const bf16*>(norm_w);
  p.eps = eps;
  p.B = B;
  p.out = static_cast<bf16*>(out);
  p.status = status;
  CUtensorMap tmS;
  if (int rc = make_tmap_f32_2d(&tmS, state, static_cast<uint64_t>(B) * G_HV * G_D, G_D, G_D, "gdn state")) return rc;
  return gdn_launch<false>(tmS, p, B, ws, ws_bytes, stream, "b200_gdn_verify");
}

extern "C" int b200_gdn_verify_replay(const void* mixed, const void* z, const void* a, const void* b, void* conv_state,
                                      const void* conv_w, void* window, const float* a_log, const float* dt_bias,
                                      const float* checkpoint, int state_slots, void* d_ring, void* dlo_ring,
                                      void* k_ring, void* klo_ring, float* g_ring, const int32_t* state_idx,
                                      const int32_t* ring_idx, const int32_t* win_idx, const int32_t* write_pos,
                                      const int32_t* cache_base, const void* norm_w, float eps, int B, void* out,
                                      void* ws, size_t ws_bytes, int32_t* status, void* stream) {
  if (!mixed || !z || !a || !b || !conv_state || !conv_w || !window || !a_log || !dt_bias || !checkpoint || !d_ring ||
      !dlo_ring || !k_ring || !klo_ring || !g_ring || !state_idx || !ring_idx || !win_idx || !write_pos || !cache_base ||
      !norm_w || !out)
    return fail(B200_E_ARG, "b200_gdn_verify_replay: null pointer");
  if (B < 0 || B > 65535 || state_slots <= 0 || state_slots > 131071)
    return fail(B200_E_ARG, "b200_gdn_verify_replay: B=%d or state_slots=%d out of range", B, state_slots);
  if (reinterpret_cast<uintptr_t>(checkpoint) & 15)
    return fail(B200_E_ALIGN, "b200_gdn_verify_replay: checkpoint must be 16-byte aligned");
  if ((reinterpret_cast<uintptr_t>(conv_w) & 7) || (reinterpret_cast<uintptr_t>(k_ring) & 7) ||
      (reinterpret_cast<uintptr_t>(window) & 3) || (reinterpret_cast<uintptr_t>(d_ring) & 15))
    return fail(B200_E_ALIGN,
                "b200_gdn_verify_replay: conv_w and k_ring must be 8-byte, window 4-byte, d_ring 16-byte aligned");
  if (B == 0) return 0;
  GdnArgs p{};
  p.mixed = static_cast<const bf16*>(mixed);
  p.z = static_cast<const bf16*>(z);
  p.a = static_cast<const bf16*>(a);
  p.b = static_cast<const bf16*>(b);
  p.conv_state = static_cast<bf16*>(conv_state);
  p.conv_w = static_cast<const bf16*>(conv_w);
  p.a_log = a_log;
  p.dt_bias = dt_bias;
  p.state = const_cast<float*>(checkpoint);  // only read in this form
  p.norm_w = static_cast<const bf16*>(norm_w);
  p.eps = eps;
  p.B = B;
  p.out = static_cast<bf16*>(out);
  p.status = status;
  p.window = static_cast<bf16*>(window);
  p.d_ring = static_cast<bf16*>(d_ring);
  p.dlo_ring = static_cast<bf16*>(dlo_ring);
  p.k_ring = static_cast<bf16*>(k_ring);
  p.klo_ring = static_cast<bf16*>(klo_ring);
  p.g_ring = g_ring;
  p.state_idx = state_idx;
  p.ring_idx = ring_idx;
  p.win_idx = win_idx;
  p.write_pos = write_pos;
  p.cache_base = cache_base;
  CUtensorMap tmS;
  if (int rc = make_tmap_f32_2d(&tmS, const_cast<float*>(checkpoint), static_cast<uint64_t>(state_slots) * G_HV * G_D, G_D,
                                G_D, "gdn checkpoint"))
    return rc;
  return gdn_launch<true>(tmS, p, B, ws, ws_bytes, stream, "b200_gdn_verify_replay");
}

extern "C" int b200_gdn_ring_fold(float* checkpoint, const void* d_ring, const void* dlo_ring, const void* k_ring,
                                  const void* klo_ring, const float* g_ring, const int32_t* state_idx,
                                  const int32_t* ring_idx, const int32_t* write_pos, const int32_t* cache_base, int B,
                                  void* stream) {
  if (!checkpoint || !d_ring || !dlo_ring || !k_ring || !klo_ring || !g_ring || !state_idx || !ring_idx || !write_pos ||
      !cache_base)
    return fail(B200_E_ARG, "b200_gdn_ring_fold: null pointer");
  if (B < 0 || B > 65535) return fail(B200_E_ARG, "b200_gdn_ring_fold: B=%d out of range", B);
  if (reinterpret_cast<uintptr_t>(checkpoint) & 15) return fail(B200_E_ALIGN, "b200_gdn_ring_fold: checkpoint must be 16-byte aligned");
  if (B == 0) return 0;
  GdnFoldArgs p{checkpoint,
                static_cast<const bf16*>(d_ring), static_cast<const bf16*>(dlo_ring), static_cast<const bf16*>(k_ring),
                static_cast<const bf16*>(klo_ring), g_ring, state_idx, ring_idx, write_pos, cache_base};
  launch_k(gdn_fold_kernel, dim3(B * G_HV), dim3(256), 0, static_cast<cudaStream_t>(stream), p);
  return launch_status("b200_gdn_ring_fold");
}
