// Expert-parallel plumbing that is not a GEMM: the barrier among the ranks of a group, the host-settable
// budget of the device-side waits, and the self-test of a wait that runs out.
//
// The reference is single-GPU (layer.py:396-402) and its device-side waits are unbounded spins
// (qk_gdn_verify.cu:140-144, qk_moe_up16.cu:656); nothing here mirrors a reference function.
#include "common.cuh"
#include "host.h"

namespace b200 {

B200_DEFINE_WAIT_BUDGET_SETTER(set_wait_budget_ep)

struct EpBarrierArgs {
  unsigned long long* flags[8];   // rank r's flag array [B200_EP_CHANNELS][8] as mapped here
  unsigned long long* epochs;     // this rank's private epochs [B200_EP_CHANNELS]
  int world, rank, channel;
  unsigned long long timeout_ns;
  int32_t* status;
};

__device__ __forceinline__ void st_release_sys(unsigned long long* p, unsigned long long v) {
  asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ unsigned long long ld_acquire_sys(const unsigned long long* p) {
  unsigned long long v;
  asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}

// One warp.  Launched with programmatic serialization: the warp may be resident while the kernel before it still runs,
// but nothing is signalled before the dependency wait has returned (that kernel complete, its stores to the peers
// performed); the kernel after it may be resident early in the same way and waits at its own top.
__global__ void __launch_bounds__(32) ep_barrier_kernel(const EpBarrierArgs a) {
  const int lane = threadIdx.x;
  pdl_wait();
  pdl_launch();
  // a rank that has already given up on a peer does not wait again (its epoch still advances, so that the
  // ranks stay in step if the host decides to carry on)
  const bool dead = a.status != nullptr && *reinterpret_cast<volatile int32_t*>(a.status) != 0;
  unsigned long long ep = 0ull;
  if (lane == 0) {
    ep = a.epochs[a.channel] + 1ull;
    a.epochs[a.channel] = ep;
  }
  ep = __shfl_sync(FULL_MASK, ep, 0);
  __threadfence_system();
  if (lane < a.world) st_release_sys(a.flags[lane] + a.channel * 8 + a.rank, ep);
  if (dead) return;
  bool late = false;
  if (lane < a.world) {
    const unsigned long long* mine = a.flags[a.rank] + a.channel * 8 + lane;
    const unsigned long long t0 = globaltimer();
    while (ld_acquire_sys(mine) < ep) {
      if (globaltimer() - t0 > a.timeout_ns) {
        late = true;
        break;
      }
    }
  }
  if (__any_sync(FULL_MASK, late) && lane == 0 && a.status) atomicCAS(a.status, 0, ST_WAIT_PEER);
  __threadfence_system();
}

// Stores `words` 4-byte words from `src` into every rank's buffer at word offset `dst_word` (an all-gather by peer
// stores: every rank puts its piece at its own offset).  grid (world, blocks): blockIdx.x = destination rank.
struct EpPutArgs {
  const uint32_t* src;
  uint32_t* dst[8];
  size_t words, dst_word;
};
__global__ void __launch_bounds__(256) ep_put_kernel(const EpPutArgs a) {
  pdl_wait();
  pdl_launch();
  uint32_t* d = a.dst[blockIdx.x] + a.dst_word;
  const size_t stride = static_cast<size_t>(gridDim.y) * 256;
  if (((reinterpret_cast<uintptr_t>(a.src) | reinterpret_cast<uintptr_t>(d)) & 15) == 0) {
    const size_t n4 = a.words >> 2;
    const uint4* s4 = reinterpret_cast<const uint4*>(a.src);
    uint4* d4 = reinterpret_cast<uint4*>(d);
    for (size_t i = blockIdx.y * 256 + threadIdx.x; i < n4; i += stride) d4[i] = s4[i];
    for (size_t i = (n4 << 2) + blockIdx.y * 256 + threadIdx.x; i < a.words; i += stride) d[i] = a.src[i];
  } else {
    for (size_t i = blockIdx.y * 256 + threadIdx.x; i < a.words; i += stride) d[i] = a.src[i];
  }
}

// A wait that cannot succeed: nothing ever arrives on the barrier.
__global__ void __launch_bounds__(32) selftest_wait_kernel(int32_t* status) {
  __shared__ uint64_t bar;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);
    abort_flag = 0;
    mbar_fence_init();
  }
  __syncwarp();
  if (threadIdx.x == 0) mbar_wait(&bar, 0u, &abort_flag, status, ST_WAIT_FULL);
}

}  // namespace b200

using namespace b200;

extern "C" int b200_ep_barrier(void* const* peer_flags_host, unsigned long long* epochs, int ep_world, int ep_rank,
                               int channel, unsigned long long timeout_ns, int32_t* status, void* stream) {
  if (!peer_flags_host || !epochs) return fail(B200_E_ARG, "b200_ep_barrier: null pointer");
  if (ep_world < 1 || ep_world > 8 || ep_rank < 0 || ep_rank >= ep_world || channel < 0 || channel >= B200_EP_CHANNELS ||
      timeout_ns == 0)
    return fail(B200_E_ARG, "b200_ep_barrier: need 1 <= ep_world <= 8, 0 <= ep_rank < ep_world, 0 <= channel < %d and a "
                "non-zero timeout (world=%d rank=%d channel=%d)", B200_EP_CHANNELS, ep_world, ep_rank, channel);
  EpBarrierArgs a{};
  for (int r = 0; r < ep_world; ++r) {
    if (!peer_flags_host[r] || (reinterpret_cast<uintptr_t>(peer_flags_host[r]) & 7))
      return fail(B200_E_ALIGN, "b200_ep_barrier: rank %d's flag array is null or not 8-byte aligned", r);
    a.flags[r] = static_cast<unsigned long long*>(peer_flags_host[r]);
  }
  a.epochs = epochs;
  a.world = ep_world;
  a.rank = ep_rank;
  a.channel = channel;
  a.timeout_ns = timeout_ns;
  a.status = status;
  launch_k(ep_barrier_kernel, dim3(1), dim3(32), 0, static_cast<cudaStream_t>(stream), a);
  return launch_status("b200_ep_barrier");
}

extern "C" int b200_ep_put(const void* src, size_t bytes, size_t dst_offset_bytes, void* const* peer_dst_host, int ep_world,
                           void* stream) {
  if (!src || !peer_dst_host) return fail(B200_E_ARG, "b200_ep_put: null pointer");
  if (ep_world < 1 || ep_world > 8 || (bytes & 3) || (dst_offset_bytes & 3) || (reinterpret_cast<uintptr_t>(src) & 3))
    return fail(B200_E_ARG, "b200_ep_put: need 1 <= ep_world <= 8 and 4-byte granularity (bytes=%zu offset=%zu)", bytes,
                dst_offset_bytes);
  if (bytes == 0) return 0;
  EpPutArgs a{};
  a.src = static_cast<const uint32_t*>(src);
  a.words = bytes >> 2;
  a.dst_word = dst_offset_bytes >> 2;
  for (int r = 0; r < ep_world; ++r) {
    if (!peer_dst_host[r] || (reinterpret_cast<uintptr_t>(peer_dst_host[r]) & 3))
      return fail(B200_E_ALIGN, "b200_ep_put: rank %d's buffer is null or not 4-byte aligned", r);
    a.dst[r] = static_cast<uint32_t*>(peer_dst_host[r]);
  }
  const size_t blocks = (a.words / 4 + 255) / 256;
  launch_k(ep_put_kernel, dim3(ep_world, static_cast<unsigned>(blocks < 1 ? 1 : (blocks > 32 ? 32 : blocks))), dim3(256), 0,
           static_cast<cudaStream_t>(stream), a);
  return launch_status("b200_ep_put");
}

extern "C" int b200_set_wait_budget_ns(unsigned long long ns) {
  if (ns == 0) ns = WAIT_BUDGET_DEFAULT_NS;
  int (*setters[])(unsigned long long) = {set_wait_budget_router, set_wait_budget_moe,        set_wait_budget_moe_fp8,
                                          set_wait_budget_attn,   set_wait_budget_attn_verify, set_wait_budget_gdn,
                                          set_wait_budget_ep};
  for (auto f : setters) {
    const int rc = f(ns);
    if (rc != 0) return fail(rc, "b200_set_wait_budget_ns: %s", cudaGetErrorString(static_cast<cudaError_t>(rc)));
  }
  return 0;
}

extern "C" int b200_selftest_wait_expiry(int32_t* status, void* stream) {
  if (!status) return fail(B200_E_ARG, "b200_selftest_wait_expiry: null pointer");
  selftest_wait_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(status);
  return launch_status("b200_selftest_wait_expiry");
}
