// Device-side helpers shared by every kernel of the library: bf16 / e4m3 conversion, bounded
// mbarrier waits, TMA (cp.async.bulk[.tensor]) issue, tcgen05 / TMEM wrappers, UMMA descriptors.
// sm_100a only.
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace b200 {

typedef __nv_bfloat16 bf16;
constexpr unsigned FULL_MASK = 0xffffffffu;

// Status codes a kernel can leave in the caller's status word (first failure wins).
enum : int {
  ST_OK = 0,
  ST_WAIT_FULL = 101,     // consumer gave up waiting for a TMA stage
  ST_WAIT_EMPTY = 102,    // producer gave up waiting for a free stage
  ST_WAIT_TMEM_FULL = 103,
  ST_WAIT_TMEM_EMPTY = 104,
  ST_WAIT_STATE = 105,    // GDN: state tile never landed
  ST_WAIT_STORE = 106,
  ST_WAIT_PEER = 107,     // expert-parallel barrier: a peer rank's flag never arrived
  ST_BAD_LIST = 110,      // routing list entry out of range (skipped)
};

// Every device-side wait is bounded: a budget of %globaltimer nanoseconds (one second unless the host changed it
// with b200_set_wait_budget_ns), after which the waiter records a status code, raises the CTA's abort flag and
// every role winds down.  The budget is a per-translation-unit device variable (the library is built without
// relocatable device code); B200_DEFINE_WAIT_BUDGET_SETTER gives each unit the host function that writes its copy.
constexpr unsigned long long WAIT_BUDGET_DEFAULT_NS = 1000ull * 1000ull * 1000ull;
static __device__ unsigned long long g_wait_budget_ns = WAIT_BUDGET_DEFAULT_NS;
#define B200_DEFINE_WAIT_BUDGET_SETTER(name)                                                              \
  int name(unsigned long long ns) {                                                                       \
    return static_cast<int>(cudaMemcpyToSymbol(b200::g_wait_budget_ns, &ns, sizeof(ns), 0, cudaMemcpyHostToDevice)); \
  }

__device__ __forceinline__ float bf2f(bf16 v) { return __bfloat162float(v); }
__device__ __forceinline__ bf16 f2bf(float v) { return __float2bfloat16_rn(v); }
__device__ __forceinline__ float rbf(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }
__device__ __forceinline__ float bf_lo(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float bf_hi(uint32_t w) { return __uint_as_float(w & 0xffff0000u); }
__device__ __forceinline__ uint32_t pack_bf2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
// two floats -> two e4m3 bytes (lo in bits 0-7), round to nearest even, saturating
__device__ __forceinline__ uint32_t e4m3x2(float lo, float hi) {
  uint16_t r;
  asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(r) : "f"(hi), "f"(lo));
  return r;
}
__device__ __forceinline__ uint32_t e4m3x4(float a, float b, float c, float d) {
  return e4m3x2(a, b) | (e4m3x2(c, d) << 16);
}

// ---- e4m3 activation quantisation of 8 bf16 values -----------------------------------------------
// scale = max(amax / 448, 1e-12), y = e4m3(x * (1 / scale)) per (row, 128-channel group): fp8.py:21-34.
__device__ __forceinline__ uint2 quant8_e4m3(const uint4 v, float inv) {
  return make_uint2(e4m3x4(bf_lo(v.x) * inv, bf_hi(v.x) * inv, bf_lo(v.y) * inv, bf_hi(v.y) * inv),
                    e4m3x4(bf_lo(v.z) * inv, bf_hi(v.z) * inv, bf_lo(v.w) * inv, bf_hi(v.w) * inv));
}
__device__ __forceinline__ float amax8(const uint4 v) {
  float a = fmaxf(fmaxf(fabsf(bf_lo(v.x)), fabsf(bf_hi(v.x))), fmaxf(fabsf(bf_lo(v.y)), fabsf(bf_hi(v.y))));
  return fmaxf(a, fmaxf(fmaxf(fabsf(bf_lo(v.z)), fabsf(bf_hi(v.z))), fmaxf(fabsf(bf_lo(v.w)), fabsf(bf_hi(v.w)))));
}

// Global stores that the compiler need not order against the C++ loads around them (no "memory" clobber): an
// epilogue that reads its row metadata from shared memory and stores through pointers it also read from there
// would otherwise reload after every store (a generic pointer may alias shared memory), one dependent
// shared-memory round trip per store.  Only for global destinations that the kernel never reads back.
__device__ __forceinline__ void st_global_na(bf16* p, bf16 v) {
  asm volatile("st.global.b16 [%0], %1;" ::"l"(__cvta_generic_to_global(p)), "h"(*reinterpret_cast<unsigned short*>(&v)));
}
__device__ __forceinline__ void st_global_na(float* p, float v) {
  asm volatile("st.global.f32 [%0], %1;" ::"l"(__cvta_generic_to_global(p)), "f"(v));
}

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ unsigned long long globaltimer() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile(
      "{\n.reg .pred p;\nelect.sync _|p, 0xffffffff;\nselp.u32 %0, 1, 0, p;\n}\n" : "=r"(pred));
  return pred != 0;
}

// ---- mbarrier --------------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}\n"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait.  `abort_flag` lives in shared memory and is shared by all roles of the CTA: the
// first waiter whose budget runs out records `code` in the caller's status word and raises it, the
// others see it on their next poll.  Returns false when the wait was abandoned.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag, int* status,
                                          int code) {
  if (mbar_try(bar, parity)) return true;
  const unsigned long long t0 = globaltimer();
  uint32_t spins = 0;
  while (true) {
    if (mbar_try(bar, parity)) return true;
    if (((++spins) & 63u) == 0u) {
      if (*abort_flag) return false;
      if (globaltimer() - t0 > g_wait_budget_ns) {
        *abort_flag = 1;
        if (status) atomicCAS(status, 0, code);
        return false;
      }
    }
  }
}

// ---- programmatic dependent launch ----
// wait: the kernels launched before this one have completed and their writes are visible (returns at once when
// the launch carried no programmatic dependency); launch: the next kernel in the stream may start.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// ---- TMA ---------------------------------------------------------------------------------------
__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(smem_u32(smem_dst)), "l"(map), "r"(x), "r"(y), "r"(smem_u32(bar))
      : "memory");
}
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, int x, int y, const void* smem_src) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%1, %2}], [%3];" ::"l"(map), "r"(x), "r"(y),
               "r"(smem_u32(smem_src))
               : "memory");
}
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(map) : "memory");
}
// plain (untiled) bulk copies: both addresses 16-byte aligned, size a multiple of 16
__device__ __forceinline__ void bulk_load(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
          smem_u32(smem_dst)),
      "l"(gsrc), "r"(bytes), "r"(smem_u32(bar))
      : "memory");
}
__device__ __forceinline__ void bulk_store(void* gdst, const void* smem_src, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(gdst), "r"(smem_u32(smem_src)),
               "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_read_all() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// ---- tcgen05 / TMEM ------------------------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_dst, uint32_t ncols) {  // whole warp
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_dst)),
               "r"(ncols)
               : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {  // whole warp
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
// arrive on an mbarrier once every MMA issued so far by this thread has completed
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void tc_mma_i8(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                          uint32_t accumulate) {
  asm volatile(
      "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n}\n" ::"r"(tmem_d),
      "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void tc_mma_tf32(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                            uint32_t accumulate) {
  asm volatile(
      "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n}\n" ::"r"(tmem_d),
      "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void tc_mma_f8(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                          uint32_t accumulate) {
  asm volatile(
      "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n}\n" ::"r"(tmem_d),
      "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}
// this warp's 32 TMEM lanes x 16 consecutive 32-bit columns
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, "
      "[%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
// this warp's 32 TMEM lanes x 32 consecutive 32-bit columns
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor for a K-major operand tile whose rows are 128 bytes long and
// were written by TMA with the 128-byte swizzle: 8-row groups are 1024 bytes apart (stride byte
// offset), the leading byte offset is unused for swizzled K-major tiles, descriptor version 1.
__device__ __forceinline__ uint64_t umma_desc_sw128(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3ffffu) >> 4);  // start address, bits [0, 14)
  d |= static_cast<uint64_t>(1) << 16;                      // leading byte offset (ignored), bits [16, 30)
  d |= static_cast<uint64_t>(1024 >> 4) << 32;              // stride byte offset, bits [32, 46)
  d |= static_cast<uint64_t>(1) << 46;                      // descriptor version (sm_100), bits [46, 48)
  d |= static_cast<uint64_t>(2) << 61;                      // layout: 128-byte swizzle, bits [61, 64)
  return d;
}
// Instruction descriptor: dense, M = 128, N = n, both operands K-major.
//   c_format bits [4,6): 1 = f32, 2 = s32;  a/b format bits [7,10) / [10,13);
//   n >> 3 in bits [17,23);  m >> 4 in bits [24,29).
__device__ __forceinline__ uint32_t umma_idesc(uint32_t c_fmt, uint32_t ab_fmt, uint32_t n) {
  return (c_fmt << 4) | (ab_fmt << 7) | (ab_fmt << 10) | ((n >> 3) << 17) | ((128u >> 4) << 24);
}
constexpr uint32_t UMMA_C_F32 = 1, UMMA_C_S32 = 2, UMMA_AB_INT8 = 1, UMMA_AB_E4M3 = 0, UMMA_AB_TF32 = 2;

}  // namespace b200
