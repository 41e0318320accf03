// Fused gated-attention projection front: fp8 block-scaled GEMM x[T,2048] . W[9216,2048]^T with the
// per-head q/k RMSNorm and the neox partial RoPE applied in the epilogue.
//
// Replaces fp8.linear_q (fp8.py:77-108; GEMM recipe qk_lt.cu:361-364) followed by
// qk_attn_verify.attn_prefill_front (qk_attn_verify.cu:765-800, norm_rope_e4m3 :180-208): the reference
// writes the bf16 projection to HBM and reads it back in a second kernel; here one head of one token
// never leaves the SM between the GEMM and the norm.
//
// Tensor-bound (154.6 GFLOP at T = 4096).  Orientation: tokens are the MMA M side (TMEM lanes), the
// 256 features of one head are the N side (TMEM columns), so a thread that owns a TMEM lane owns a
// whole token row of the head and the RMS reduction stays thread-local.  Tile = 128 tokens x 256
// features x K 128 per stage; per 128-k block the chain starts from zero in one of two TMEM partial
// buffers (2 x 256 columns = all of TMEM) and eight epilogue warps promote it into registers,
// acc = fma(partial, a_scale[token] * w_scale[block], acc): two warps share a lane quadrant and take
// 128 columns each, which is exactly one weight scale block, so the scale is one scalar per thread
// and k block.
#include "common.cuh"
#include "host.h"

namespace b200 {

B200_DEFINE_WAIT_BUDGET_SETTER(set_wait_budget_attn)

constexpr int AT_H = 2048, AT_HD = 256, AT_HQ = 16, AT_HKV = 2, AT_ROT = 64;
constexpr int AT_NCOLS = AT_HQ * 2 * AT_HD + 2 * AT_HKV * AT_HD;  // 9216
constexpr int AT_NT = AT_NCOLS / AT_HD;                           // 36 head tiles
constexpr int AT_KS = AT_H / 128;                                 // 16
constexpr int AT_THREADS = 320;                                   // TMA warp, MMA warp, 8 epilogue warps
constexpr int AT_A = 128 * 128, AT_B = 256 * 128, AT_STAGE = AT_A + AT_B, AT_STAGES = 4;
constexpr int AT_META = 2 * 2 * 128 * 4 /*ss halves, two phases*/ + 2 * 256 * 4 /*1 + w*/;
constexpr int AT_SCALES = 8 * (32 * AT_KS + AT_KS) * 4;  // per epilogue warp: its 32 tokens' activation scales + one weight scale row
constexpr int AT_SMEM = AT_STAGES * AT_STAGE + 1024 + 256 + AT_META + AT_SCALES;

struct AttnArgs {
  const float* a_scale;   // [T, 16]
  const float* w_s;       // [72, 16]
  const bf16* q_norm_w;   // [256]
  const bf16* k_norm_w;   // [256]
  const int64_t* positions;
  const float* cos_sin;   // [max_pos, 64]
  int max_pos;
  float eps;
  int T, out_fp8;
  void* q;     // [T,16,256]
  bf16* gate;  // [T,16,256]
  void* k;     // [T,2,256]
  void* v;     // [T,2,256]
  int32_t* status;
};

// two fp32 FMAs in one instruction (each lane an IEEE fma, same results as two fmaf)
__device__ __forceinline__ void fma2(float& a0, float& a1, float x0, float x1, float s) {
  unsigned long long acc, x, sc;
  asm("mov.b64 %0, {%1, %2};" : "=l"(acc) : "f"(a0), "f"(a1));
  asm("mov.b64 %0, {%1, %2};" : "=l"(x) : "f"(x0), "f"(x1));
  asm("mov.b64 %0, {%1, %1};" : "=l"(sc) : "f"(s));
  asm("fma.rn.f32x2 %0, %1, %2, %0;" : "+l"(acc) : "l"(x), "l"(sc));
  asm("mov.b64 {%0, %1}, %2;" : "=f"(a0), "=f"(a1) : "l"(acc));
}
__device__ __forceinline__ void at_cp16(void* smem_dst, const void* gsrc) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 16;" ::"r"(smem_u32(smem_dst)), "l"(gsrc) : "memory");
}

__global__ void __launch_bounds__(AT_THREADS, 1)
attn_front_kernel(const __grid_constant__ CUtensorMap tmX, const __grid_constant__ CUtensorMap tmW, const AttnArgs p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + AT_STAGES * AT_STAGE);
  uint64_t* empty = full + AT_STAGES;
  uint64_t* pfull = empty + AT_STAGES;  // [2]
  uint64_t* pempty = pfull + 2;         // [2]
  uint64_t* ssbar = pempty + 2;         // [1] both column halves have published their sum of squares
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(ssbar + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  float* m_ss = reinterpret_cast<float*>(smem + AT_STAGES * AT_STAGE + 256);  // [2 phases][2 halves][128]
  float* m_w1 = m_ss + 512;                                                    // [2][256]: 1 + q_norm_w, 1 + k_norm_w

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int s = 0; s < AT_STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&pfull[b], 1);
      mbar_init(&pempty[b], 8);
    }
    mbar_init(ssbar, 256);
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmX);
    tma_prefetch_desc(&tmW);
  }
  for (int i = threadIdx.x; i < 512; i += AT_THREADS)
    m_w1[i] = 1.f + bf2f(i < 256 ? p.q_norm_w[i] : p.k_norm_w[i - 256]);
  if (warp == 1) tmem_alloc(tmem_slot, 512);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const int mtiles = (p.T + 127) / 128;
  const int ntiles = mtiles * AT_NT;

  if (warp == 0) {
    if (lane == 0) {  // ---------------- TMA producer ----------------
      int stage = 0, issued = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; ok && tile < ntiles; tile += gridDim.x) {
        const int j = tile / mtiles, mt = tile - j * mtiles;
        for (int ks = 0; ks < AT_KS; ++ks) {
          if (!mbar_wait(&empty[stage], phase ^ 1u, abort_flag, p.status, ST_WAIT_EMPTY)) {
            ok = false;
            break;
          }
          uint8_t* sA = smem + stage * AT_STAGE;
          mbar_expect_tx(&full[stage], AT_STAGE);
          tma_load_2d(sA, &tmX, ks * 128, mt * 128, &full[stage]);
          tma_load_2d(sA + AT_A, &tmW, ks * 128, j * 256, &full[stage]);
          tma_load_2d(sA + AT_A + AT_A, &tmW, ks * 128, j * 256 + 128, &full[stage]);
          ++issued;
          if (++stage == AT_STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
      if (!ok) {
        const unsigned long long t0 = globaltimer();
        const int back = issued < AT_STAGES ? issued : AT_STAGES;
        for (int i = 1; i <= back; ++i) {
          int s = stage - i;
          uint32_t ph = phase;
          if (s < 0) {
            s += AT_STAGES;
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
      uint32_t phase = 0, g = 0;
      const uint32_t idesc = umma_idesc(UMMA_C_F32, UMMA_AB_E4M3, 256);
      bool ok = true;
      for (int tile = blockIdx.x; ok && tile < ntiles; tile += gridDim.x) {
        for (int ks = 0; ks < AT_KS; ++ks, ++g) {
          const uint32_t pb = g & 1u, pphase = (g >> 1) & 1u;
          if (!mbar_wait(&pempty[pb], pphase ^ 1u, abort_flag, p.status, ST_WAIT_TMEM_EMPTY) ||
              !mbar_wait(&full[stage], phase, abort_flag, p.status, ST_WAIT_FULL)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sA = smem_u32(smem + stage * AT_STAGE);
          const uint32_t sB = sA + AT_A;
#pragma unroll
          for (int kk = 0; kk < 4; ++kk)
            tc_mma_f8(tmem_base + pb * 256, umma_desc_sw128(sA + kk * 32), umma_desc_sw128(sB + kk * 32), idesc, kk != 0);
          tc_commit(&empty[stage]);
          tc_commit(&pfull[pb]);
          if (++stage == AT_STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
    }
  } else {
    // ---------------- promotion + fused epilogue: warps 2..9 ----------------
    const int q = warp & 3;               // TMEM lane quadrant
    const int hh = (warp - 2) >> 2;       // column half of the head: 0 -> features 0..127, 1 -> 128..255
    const int row = q * 32 + lane;        // token row inside the tile
    uint32_t g = 0, sscount = 0;
    bool ok = true;
    // This warp's scales of a tile (its 32 tokens' 16 activation scales, the 16 weight block scales of its 128
    // columns) are copied into shared memory asynchronously when the previous tile's k loop has ended, under that
    // tile's epilogue: with the operand stream in flight a global load on the critical path costs microseconds.
    float* m_as = reinterpret_cast<float*>(smem + AT_STAGES * AT_STAGE + 256 + AT_META) + (warp - 2) * (32 * AT_KS + AT_KS);
    float* m_ws = m_as + 32 * AT_KS;
    auto fetch_scales = [&](int tile) {
      if (tile >= ntiles) return;
      const int j = tile / mtiles, mt = tile - j * mtiles;
      const int t = mt * 128 + row;
      const float* asrow = p.a_scale + static_cast<size_t>(t < p.T ? t : 0) * AT_KS;
#pragma unroll
      for (int c = 0; c < AT_KS / 4; ++c) at_cp16(m_as + lane * AT_KS + 4 * c, asrow + 4 * c);
      if (lane < AT_KS / 4) at_cp16(m_ws + 4 * lane, p.w_s + static_cast<size_t>(2 * j + hh) * AT_KS + 4 * lane);
      asm volatile("cp.async.commit_group;" ::: "memory");
    };
    fetch_scales(blockIdx.x);
    for (int tile = blockIdx.x; ok && tile < ntiles; tile += gridDim.x) {
      const int j = tile / mtiles, mt = tile - j * mtiles;
      const int t = mt * 128 + row;
      asm volatile("cp.async.wait_group 0;" ::: "memory");
      __syncwarp();
      float acc[128];
#pragma unroll
      for (int c = 0; c < 128; ++c) acc[c] = 0.f;
      for (int ks = 0; ks < AT_KS; ++ks, ++g) {
        const uint32_t pb = g & 1u, pphase = (g >> 1) & 1u;
        const float sc = __fmul_rn(m_as[lane * AT_KS + ks], m_ws[ks]);
        if (!mbar_wait(&pfull[pb], pphase, abort_flag, p.status, ST_WAIT_TMEM_FULL)) {
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t taddr = tmem_base + pb * 256 + hh * 128 + (static_cast<uint32_t>(q * 32) << 16);
#pragma unroll
        for (int c0 = 0; c0 < 128; c0 += 32) {
          uint32_t r[32];
          tmem_ld32(taddr + c0, r);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; i += 2)
            fma2(acc[c0 + i], acc[c0 + i + 1], __uint_as_float(r[i]), __uint_as_float(r[i + 1]), sc);
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&pempty[pb]);
      }
      if (!ok) break;
      __syncwarp();
      fetch_scales(tile + gridDim.x);  // lands during this tile's epilogue
      // ---- epilogue on the thread's 128 features of token t ----
      const bool is_q = j < 2 * AT_HQ && (j & 1) == 0;
      const bool is_gate = j < 2 * AT_HQ && (j & 1) == 1;
      const bool is_k = j >= 2 * AT_HQ && j < 2 * AT_HQ + AT_HKV;
      const int head = j < 2 * AT_HQ ? (j >> 1) : (is_k ? j - 2 * AT_HQ : j - 2 * AT_HQ - AT_HKV);
#pragma unroll
      for (int c = 0; c < 128; ++c) acc[c] = rbf(acc[c]);  // the projection is stored as bf16 before the front
      if (is_q || is_k) {
        float ss = 0.f;
#pragma unroll
        for (int c = 0; c < 128; ++c) ss = fmaf(acc[c], acc[c], ss);
        float* ssb = m_ss + (sscount & 1u) * 256;  // two phases: a fast thread may already write the next tile's
        ssb[hh * 128 + row] = ss;
        mbar_arrive(ssbar);
        if (!mbar_wait(ssbar, sscount & 1u, abort_flag, p.status, ST_WAIT_STORE)) break;
        ++sscount;
        const float tot = ssb[row] + ssb[128 + row];
        const float inv = rsqrtf(tot / AT_HD + p.eps);
        const float* w1 = m_w1 + (is_k ? 256 : 0) + hh * 128;
#pragma unroll
        for (int c = 0; c < 128; ++c) acc[c] = rbf(acc[c] * inv * w1[c]);
        if (hh == 0 && t < p.T) {
          long long pos = p.positions[t];
          pos = pos < 0 ? 0 : (pos >= p.max_pos ? p.max_pos - 1 : pos);
          const float* cs = p.cos_sin + static_cast<size_t>(pos) * AT_ROT;
#pragma unroll
          for (int i = 0; i < AT_ROT / 2; ++i) {
            const float cv = cs[i], sv = cs[AT_ROT / 2 + i];
            const float lo = acc[i], hi = acc[i + AT_ROT / 2];
            acc[i] = rbf(__fmul_rn(lo, cv) - __fmul_rn(hi, sv));
            acc[i + AT_ROT / 2] = rbf(__fmul_rn(hi, cv) + __fmul_rn(lo, sv));
          }
        }
      }
      if (t < p.T) {
        if (is_gate) {
          uint4* dst = reinterpret_cast<uint4*>(p.gate + (static_cast<size_t>(t) * AT_HQ + head) * AT_HD + hh * 128);
#pragma unroll
          for (int c = 0; c < 128; c += 8)
            dst[c >> 3] = make_uint4(pack_bf2(acc[c], acc[c + 1]), pack_bf2(acc[c + 2], acc[c + 3]),
                                     pack_bf2(acc[c + 4], acc[c + 5]), pack_bf2(acc[c + 6], acc[c + 7]));
        } else {
          void* base = is_q ? p.q : (is_k ? p.k : p.v);
          const int heads = is_q ? AT_HQ : AT_HKV;
          const size_t off = (static_cast<size_t>(t) * heads + head) * AT_HD + hh * 128;
          if (p.out_fp8) {
            uint4* dst = reinterpret_cast<uint4*>(static_cast<uint8_t*>(base) + off);
#pragma unroll
            for (int c = 0; c < 128; c += 16)
              dst[c >> 4] = make_uint4(e4m3x4(acc[c], acc[c + 1], acc[c + 2], acc[c + 3]),
                                       e4m3x4(acc[c + 4], acc[c + 5], acc[c + 6], acc[c + 7]),
                                       e4m3x4(acc[c + 8], acc[c + 9], acc[c + 10], acc[c + 11]),
                                       e4m3x4(acc[c + 12], acc[c + 13], acc[c + 14], acc[c + 15]));
          } else {
            uint4* dst = reinterpret_cast<uint4*>(static_cast<bf16*>(base) + off);
#pragma unroll
            for (int c = 0; c < 128; c += 8)
              dst[c >> 3] = make_uint4(pack_bf2(acc[c], acc[c + 1]), pack_bf2(acc[c + 2], acc[c + 3]),
                                       pack_bf2(acc[c + 4], acc[c + 5]), pack_bf2(acc[c + 6], acc[c + 7]));
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

}  // namespace b200

using namespace b200;

extern "C" size_t b200_attn_front_workspace_bytes(int T) {
  if (T <= 0) return 0;
  auto up = [](size_t v) { return (v + 1023) & ~size_t(1023); };
  return up(static_cast<size_t>(T) * AT_H) + up(static_cast<size_t>(T) * AT_KS * 4);
}

// `x` bf16 rows quantised here into `ws`, or (x == nullptr) rows that arrive as e4m3 `xq_in` + scales `xs_in`
static int attn_front_impl(const void* x, const void* xq_in, const float* xs_in, int T, const void* w, const float* w_s,
                           const void* q_norm_w, const void* k_norm_w, const int64_t* positions, const float* cos_sin,
                           int max_pos, float eps, int out_fp8, void* q, void* gate, void* k, void* v, void* ws,
                           size_t ws_bytes, int32_t* status, void* stream) {
  const bool pre = x == nullptr;
  if ((!pre && !ws) || (pre && (!xq_in || !xs_in)) || !w || !w_s || !q_norm_w || !k_norm_w || !positions || !cos_sin || !q ||
      !gate || !k || !v)
    return fail(B200_E_ARG, "b200_attn_front: null pointer");
  if (T <= 0 || max_pos <= 0) return fail(B200_E_ARG, "b200_attn_front: bad shape (T=%d max_pos=%d)", T, max_pos);
  if (!pre && ws_bytes < b200_attn_front_workspace_bytes(T))
    return fail(B200_E_WS, "b200_attn_front: workspace %zu < %zu bytes", ws_bytes, b200_attn_front_workspace_bytes(T));
  if (!pre && (reinterpret_cast<uintptr_t>(ws) & 1023))
    return fail(B200_E_ALIGN, "b200_attn_front: workspace must be 1024-byte aligned");
  if ((reinterpret_cast<uintptr_t>(pre ? xq_in : x) | reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(gate) |
       reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(v) | reinterpret_cast<uintptr_t>(cos_sin)) & 15)
    return fail(B200_E_ALIGN, "b200_attn_front: x, q, gate, k, v and cos_sin must be 16-byte aligned");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const uint8_t* xq = pre ? static_cast<const uint8_t*>(xq_in) : static_cast<uint8_t*>(ws);
  const float* xs = pre ? xs_in
                        : reinterpret_cast<float*>(static_cast<uint8_t*>(ws) +
                                                   ((static_cast<size_t>(T) * AT_H + 1023) & ~size_t(1023)));
  CUtensorMap tmX, tmW;
  int rc;
  if ((rc = make_tmap_bytes_2d(&tmX, xq, T, AT_H, 128, "attn activations"))) return rc;
  if ((rc = make_tmap_bytes_2d(&tmW, w, AT_NCOLS, AT_H, 128, "attn weight"))) return rc;
  static DeviceOnce once;
  once.run([] { cudaFuncSetAttribute(attn_front_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, AT_SMEM); });
  if (!pre) b200::b200_quant_rows_f8_launch(x, T, AT_H, const_cast<uint8_t*>(xq), const_cast<float*>(xs), st);
  AttnArgs a{xs, w_s, static_cast<const bf16*>(q_norm_w), static_cast<const bf16*>(k_norm_w), positions, cos_sin,
             max_pos, eps, T, out_fp8, q, static_cast<bf16*>(gate), k, v, status};
  const int ntiles = ((T + 127) / 128) * AT_NT;
  const int grid = ntiles < sm_count() ? ntiles : sm_count();
  attn_front_kernel<<<grid, AT_THREADS, AT_SMEM, st>>>(tmX, tmW, a);
  return launch_status("b200_attn_front");
}

extern "C" int b200_attn_front(const void* x, int T, const void* w, const float* w_s, const void* q_norm_w,
                               const void* k_norm_w, const int64_t* positions, const float* cos_sin, int max_pos,
                               float eps, int out_fp8, void* q, void* gate, void* k, void* v, void* ws,
                               size_t ws_bytes, int32_t* status, void* stream) {
  if (!x) return fail(B200_E_ARG, "b200_attn_front: null pointer");
  return attn_front_impl(x, nullptr, nullptr, T, w, w_s, q_norm_w, k_norm_w, positions, cos_sin, max_pos, eps, out_fp8, q,
                         gate, k, v, ws, ws_bytes, status, stream);
}

extern "C" int b200_attn_front_q(const void* xq, const float* xs, int T, const void* w, const float* w_s,
                                 const void* q_norm_w, const void* k_norm_w, const int64_t* positions,
                                 const float* cos_sin, int max_pos, float eps, int out_fp8, void* q, void* gate, void* k,
                                 void* v, int32_t* status, void* stream) {
  return attn_front_impl(nullptr, xq, xs, T, w, w_s, q_norm_w, k_norm_w, positions, cos_sin, max_pos, eps, out_fp8, q, gate,
                         k, v, nullptr, 0, status, stream);
}
