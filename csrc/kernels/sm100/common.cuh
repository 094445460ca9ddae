// Shared device-side helpers for the sm_100a kernels: PTX wrappers for mbarrier, TMA
// (cp.async.bulk.tensor into this CTA's own shared memory only), tcgen05 (TMEM alloc, MMA, commit, ld),
// bounded waits with a sticky error word, and small numeric utilities.
//
// Every wait in this tree is bounded: a wait that runs out records a code in the launch's
// error word and the kernel unwinds normally (frees TMEM, returns), so a failed peer or a
// programming error never leaves a GPU spinning.
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>

#define KERN_DEVICE __device__ __forceinline__

namespace kern {

// ---- error codes written to the error word (first writer wins) ------------------------------
enum : int {
  ERR_NONE = 0,
  ERR_WAIT_FULL = 101,      // consumer gave up waiting for a TMA stage
  ERR_WAIT_EMPTY = 102,     // producer gave up waiting for a free stage
  ERR_WAIT_TMEM_FULL = 103, // epilogue gave up waiting for an accumulator
  ERR_WAIT_TMEM_EMPTY = 104,// MMA gave up waiting for a drained accumulator
  ERR_WAIT_PEER = 200,      // + rank: a peer flag never arrived
  ERR_BOUNDS = 300,         // a checked index was out of range (access skipped)
};

KERN_DEVICE void set_error(int* err, int code) {
  if (err != nullptr) atomicCAS(err, 0, code);
}

// ---- checked builds -------------------------------------------------------------------------
// With -DKERN_CHECKED every module carries a table of the address ranges the runtime allocated or mapped (sorted by
// base, filled when the programs are compiled and again when peers connect). KERN_CHECK(p, bytes, site) is then a
// binary search: an access of `bytes` at `p` that lies in no range is recorded (first one wins: site and address) and
// the macro is false, so the caller skips the access instead of faulting. The sites are the accesses whose address
// comes from data — a token id, a slot, a page, a permutation entry, a peer table. Without the define the macro is
// the constant true and the table does not exist. An empty table (the module loaded by something other than the
// runtime) passes everything.
#ifdef KERN_CHECKED
}  // namespace kern
extern "C" {
__device__ unsigned long long kern_spans[2 * 2048];
__device__ int kern_span_count;
__device__ unsigned long long kern_check_fail[2];
}
namespace kern {
__device__ __noinline__ bool checked_access(const void* p, unsigned long long bytes, int site) {
  const unsigned long long a = reinterpret_cast<unsigned long long>(p);
  const int n = kern_span_count;
  if (n == 0) return true;
  int lo = 0, hi = n;                      // the last range whose base is <= a
  while (lo < hi) {
    const int mid = (lo + hi) >> 1;
    if (kern_spans[2 * mid] <= a) lo = mid + 1; else hi = mid;
  }
  if (lo > 0 && a + bytes <= kern_spans[2 * (lo - 1) + 1]) return true;
  if (atomicCAS(&kern_check_fail[0], 0ull, ((unsigned long long)site << 32) | 1ull) == 0ull) kern_check_fail[1] = a;
  return false;
}
#define KERN_CHECK(p, bytes, site) ::kern::checked_access((p), (bytes), (site))
#else
#define KERN_CHECK(p, bytes, site) true
#endif
// check sites
enum : int {
  SITE_EMBED_ROW = 1,       // embedding row of a token id
  SITE_KV_APPEND = 2,       // the cache row a new token's K / V go to
  SITE_MOE_GATHER = 3,      // expert-sorted row written from a permutation entry
  SITE_MOE_COMBINE = 4,     // expert-sorted row read back through the permutation
  SITE_EP_PULL = 5,         // a routed row pulled from its home rank
  SITE_EP_SLOT = 6,         // a result row stored into its (token, choice) slot
  SITE_STATE_SLOT = 7,      // a per-sequence recurrent state addressed by slot
  SITE_LATENT_ROW = 8,      // a latent cache row addressed through a page table
};

// ---- address helpers ------------------------------------------------------------------------
KERN_DEVICE uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// ---- mbarrier -------------------------------------------------------------------------------
KERN_DEVICE void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
KERN_DEVICE void mbar_fence_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
KERN_DEVICE void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)),
               "r"(bytes)
               : "memory");
}
KERN_DEVICE void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
KERN_DEVICE uint32_t mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok;
}
// Bounded wait. Returns false after `limit` polls (each poll is itself a short hardware wait).
// `abort_flag` is a CTA-shared word: once any role gives up, every other wait returns at once.
KERN_DEVICE bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag,
                           uint32_t limit = (1u << 24)) {
  for (uint32_t i = 0; i < limit; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((i & 0xff) == 0xff && *abort_flag != 0) return false;
  }
  return false;
}

// The same wait bounded by wall-clock time instead of a poll count (a poll's own duration is up to the hardware, so a
// count of polls can be minutes): gives up `limit_ns` after its first miss.
KERN_DEVICE uint64_t globaltimer_ns();
KERN_DEVICE bool mbar_wait_ns(uint64_t* bar, uint32_t parity, volatile int* abort_flag, uint64_t limit_ns = 2000000000ull) {
  if (mbar_try_wait(bar, parity)) return true;
  const uint64_t t0 = globaltimer_ns();
  for (uint32_t i = 0;; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((i & 0x3f) == 0x3f) {
      if (*abort_flag != 0) return false;
      if (globaltimer_ns() - t0 > limit_ns) return false;
    }
  }
}

// ---- TMA (tiled bulk tensor copies, each into the issuing CTA only) -------------------------------
KERN_DEVICE void tma_prefetch_desc(const CUtensorMap* m) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(m)) : "memory");
}
KERN_DEVICE void tma_load_2d(void* dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%2, %3}], [%4];" ::"r"(smem_u32(dst)),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(smem_u32(bar))
      : "memory");
}
KERN_DEVICE void tma_load_3d(void* dst, const CUtensorMap* map, int x, int y, int z,
                             uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%2, %3, %4}], [%5];" ::"r"(smem_u32(dst)),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(z), "r"(smem_u32(bar))
      : "memory");
}
KERN_DEVICE void tma_store_2d(const CUtensorMap* map, const void* src, int x, int y) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.tile.bulk_group [%0, {%2, %3}], [%1];" ::
                   "l"(reinterpret_cast<uint64_t>(map)),
               "r"(smem_u32(src)), "r"(x), "r"(y)
               : "memory");
}
KERN_DEVICE void tma_store_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
KERN_DEVICE void tma_store_wait_all() {
  asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
}
KERN_DEVICE void tma_store_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
}
KERN_DEVICE void fence_proxy_async() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
// 1-D bulk copy global -> shared (16-byte aligned addresses and size), completes on an mbarrier.
KERN_DEVICE void bulk_load_1d(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::
          "r"(smem_u32(dst)),
      "l"(reinterpret_cast<uint64_t>(src)), "r"(bytes), "r"(smem_u32(bar))
      : "memory");
}

// ---- tcgen05 / TMEM ---------------------------------------------------------------------------
// Allocate `ncols` (power of two, 32..512) TMEM columns; the base address lands in *dst (shared).
// Warp-collective: all 32 lanes of one warp call it.
KERN_DEVICE void tmem_alloc(uint32_t* dst_smem, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                   smem_u32(dst_smem)),
               "r"(ncols)
               : "memory");
}
KERN_DEVICE void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
KERN_DEVICE void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols)
               : "memory");
}
KERN_DEVICE void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
KERN_DEVICE void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
// Arrive once on `bar` when every tcgen05.mma issued so far by this thread has completed.
KERN_DEVICE void tc_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                   smem_u32(bar))
               : "memory");
}

// Shared-memory matrix descriptor for a K-major tile whose rows are 128 bytes, written by TMA with
// the 128-byte swizzle: 8-row groups are 1024 bytes apart (stride byte offset), the leading byte
// offset is unused for swizzled K-major operands, descriptor version 1 (Blackwell), layout type 2
// (SWIZZLE_128B). The tile base must be 1024-byte aligned; stepping along K inside the 128-byte
// row adds the byte offset to the start address.
KERN_DEVICE uint64_t umma_desc_sw128(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3FFFF) >> 4);   // start address, bits [0,14)
  d |= (uint64_t)0 << 16;                         // leading byte offset (unused)
  d |= (uint64_t)(1024 >> 4) << 32;               // stride byte offset, bits [32,46)
  d |= (uint64_t)1 << 46;                         // descriptor version
  d |= (uint64_t)2 << 61;                         // SWIZZLE_128B
  return d;
}

// Instruction descriptor for kind::f16 with bf16 A/B (both K-major), f32 accumulate.
KERN_DEVICE constexpr uint32_t umma_idesc_bf16(int m, int n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) |
         ((uint32_t)(m >> 4) << 24);
}
// D[tmem] (+)= A[smem] * B[smem]^T ; issued by ONE thread.
KERN_DEVICE void umma_bf16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                           uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// kind::f8f6f4: e4m3 x e4m3 (or other 8/6/4-bit formats) -> f32, dense, K = 32 per instruction.
KERN_DEVICE void umma_f8f6f4(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                             uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// Load 32 consecutive f32 columns of this thread's TMEM lane (warp w reads lanes 32*(w%4)..+31).
KERN_DEVICE void tmem_ld_32x32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]),
        "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]),
        "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
KERN_DEVICE void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// ---- programmatic dependent launch --------------------------------------------------------------
// Only reads of weights / descriptors may precede pdl_wait() in a kernel launched with the
// programmatic-stream-serialization attribute.
KERN_DEVICE void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
KERN_DEVICE void pdl_launch_dependents() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

// ---- numerics -----------------------------------------------------------------------------------
KERN_DEVICE float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
KERN_DEVICE float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
KERN_DEVICE uint32_t pack_bf16x2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
KERN_DEVICE float2 unpack_bf16x2(uint32_t u) {
  __nv_bfloat162 v = *reinterpret_cast<__nv_bfloat162*>(&u);
  return __bfloat1622float2(v);
}
KERN_DEVICE float silu(float x) { return x / (1.0f + __expf(-x)); }

// system-scope acquire / release for flags that another GPU writes
KERN_DEVICE void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
KERN_DEVICE uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
KERN_DEVICE uint64_t globaltimer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

}  // namespace kern
