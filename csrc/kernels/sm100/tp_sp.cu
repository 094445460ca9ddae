// Sequence-parallel half of a tensor-parallel decoder layer: the reduce side of the GEMM + reduce-scatter, fused with
// the residual add and the RMSNorm, on the rows this rank owns only.
//
// Layout. Rows are owned in sub-blocks of 32: sub-block s belongs to rank s % nranks, at dense index
// (s / nranks) * 32 + row % 32 of that rank's staging slots. The o / down projection before this kernel is the
// tensor-parallel GEMM whose epilogue pushed every partial row over NVLink into its owner's slot of the pushing rank
// (tp_gemm.cu, grid = 0 form). This kernel, on the owner:
//   x[row] += sum over ranks of slot[r][idx]        (fp32 sum, one rounding)
//   g[row]  = rmsnorm(x[row]) * w                   (g: the all-gather buffer the next GEMM pulls from)
// The all-gather half comes in two forms. Pull (g_peers null): nothing is sent back, the QKV / gate-up GEMM that follows
// pulls the rows it needs out of every owner's g while its own tiles run (ag_gemm.cu, `_sp` entries). Push (g_peers set):
// the owner writes each normed row straight into every rank's g — posted stores keep the link far busier than loads
// issued from the SMs do — and the following GEMM only waits for the owners' "rows final" flags. Either way the link
// carries (n-1)/n of the message once in each direction per layer, and the norm / residual work is 1/n of the
// replicated layout's.
//
// Synchronisation, all by epoch words that only grow (captured graphs replay without host help):
//   flags[0][r]  "rank r has launched this call's reduce kernel": written by r on every peer at kernel start — r's GEMM
//                before it has completed, so r's pushes are visible. Every CTA waits for all of them (bounded).
//   flags[1][r]  "rank r's rows of g are final for this call": written by the last CTA of r to finish.
//   state[0]     this rank's epoch (calls so far); state[1] counts finished CTAs of the running call.
// The arrival wait also lines the ranks up once per call, which is what lets g, x and the staging slots be reused
// call after call without a barrier kernel: nobody can be more than one call ahead of the slowest rank.
// Every wait is bounded by timeout_ns of %globaltimer; a wait that runs out records 200 + rank and the kernel returns.
//
// Reference counterpart: docs/multi-gpu.md:495-528 describes the layout (reduce-scatter, norm on own rows, all-gather)
// as NCCL calls between library GEMMs; there is no fused kernel for it there.
#include "common.cuh"

using namespace kern;

namespace {
constexpr int kThreads = 256;
constexpr int kSub = 32;   // rows per ownership sub-block (kSpRows in gemm_bf16.cu)
constexpr int kFlagStride = 32;   // words per flag row: at most 32 ranks

KERN_DEVICE void add8(float (&acc)[8], uint4 v) {
  float2 a = unpack_bf16x2(v.x), b = unpack_bf16x2(v.y), c = unpack_bf16x2(v.z), d = unpack_bf16x2(v.w);
  acc[0] += a.x; acc[1] += a.y; acc[2] += b.x; acc[3] += b.y;
  acc[4] += c.x; acc[5] += c.y; acc[6] += d.x; acc[7] += d.y;
}
KERN_DEVICE uint4 pack8(const float (&f)[8]) {
  uint4 o;
  o.x = pack_bf16x2(f[0], f[1]); o.y = pack_bf16x2(f[2], f[3]);
  o.z = pack_bf16x2(f[4], f[5]); o.w = pack_bf16x2(f[6], f[7]);
  return o;
}
// peer stores land in this GPU's memory behind the back of its L1: read them with a volatile load
KERN_DEVICE uint4 ld_volatile16(const void* p) {
  uint4 v;
  asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}
KERN_DEVICE bool wait_epoch(const uint32_t* flag, uint32_t epoch, long long timeout_ns) {
  const uint64_t t0 = globaltimer_ns();
  while ((int32_t)(ld_acquire_sys(flag) - epoch) < 0) {     // epochs wrap after 2^32 calls: signed distance
    if ((long long)(globaltimer_ns() - t0) > timeout_ns) return false;
    __nanosleep(20);
  }
  return true;
}
}  // namespace

// grid: any (the same on every launch of one rank is not required), block 256 (eight rows at a time, a warp each).
//   comm  : [2 parities][nranks][slot_rows][hidden] bf16 (exported; written by the peers' GEMM epilogues)
//   flags : [2][32] u32 (exported, zero at start; row 0 arrivals, row 1 "rows final");  state: [2] u32 local, zero at start
extern "C" __global__ void __launch_bounds__(kThreads)
    kern_sp_reduce_norm(__nv_bfloat16* x, __nv_bfloat16* g, const __nv_bfloat16* w, const __nv_bfloat16* comm,
                        uint32_t* flags, const unsigned long long* flag_peers, uint32_t* state, int* err, int rank,
                        int nranks, int rows, int hidden, int slot_rows, float eps, int plus_one, long long timeout_ns,
                        const unsigned long long* g_peers) {
  __shared__ int failed;
  pdl_wait();
  if (threadIdx.x == 0) failed = (err != nullptr && *reinterpret_cast<volatile int*>(err) != 0) ? 1 : 0;
  const uint32_t epoch = *reinterpret_cast<volatile uint32_t*>(state) + 1;
  __syncthreads();
  if (blockIdx.x == 0 && (int)threadIdx.x < nranks)
    st_release_sys(reinterpret_cast<uint32_t*>(flag_peers[threadIdx.x]) + rank, epoch);
  if ((int)threadIdx.x < nranks && !failed) {
    if (!wait_epoch(flags + threadIdx.x, epoch, timeout_ns)) {
      set_error(err, ERR_WAIT_PEER + threadIdx.x);
      failed = 1;
    }
  }
  __syncthreads();

  const int nv = hidden / 8;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const size_t slot_elems = (size_t)slot_rows * hidden;
  const __nv_bfloat16* mine = comm + (size_t)(epoch & 1) * nranks * slot_elems;
  const int subs = (rows + kSub - 1) / kSub;                         // sub-blocks of the call
  const int my_subs = subs > rank ? (subs - rank + nranks - 1) / nranks : 0;
  const int my_rows = my_subs * kSub;                                // dense indices 0 .. my_rows-1 (the tail may be past `rows`)
  if (!failed) {
    // one warp per row, no block-wide synchronisation: a lane owns vectors lane, lane + 32, ... of the row in both
    // passes (sum + residual, then the norm over the row it has just written), four vectors of every slot in flight
    for (int idx = blockIdx.x * (kThreads / 32) + warp; idx < my_rows; idx += gridDim.x * (kThreads / 32)) {
      const int row = ((idx / kSub) * nranks + rank) * kSub + idx % kSub;
      if (row >= rows) continue;
      if (idx >= slot_rows) { if (lane == 0) set_error(err, ERR_BOUNDS); continue; }
      uint4* xr = reinterpret_cast<uint4*>(x + (size_t)row * hidden);
      const uint4* part = reinterpret_cast<const uint4*>(mine + (size_t)idx * hidden);
      const size_t slot_vecs = slot_elems / 8;
      float ss = 0.f;
      for (int v0 = lane; v0 < nv; v0 += 128) {
        float acc[4][8];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
#pragma unroll
          for (int e = 0; e < 8; ++e) acc[u][e] = 0.f;
          const int v = v0 + 32 * u;
          if (v < nv) add8(acc[u], xr[v]);
        }
        for (int r = 0; r < nranks; ++r) {   // rank order
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            const int v = v0 + 32 * u;
            if (v < nv) add8(acc[u], ld_volatile16(part + r * slot_vecs + v));
          }
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int v = v0 + 32 * u;
          if (v < nv) {
            const uint4 out = pack8(acc[u]);
            xr[v] = out;
            float f[8] = {0, 0, 0, 0, 0, 0, 0, 0};
            add8(f, out);                    // the norm sees the rounded residual stream, as the unfused layer would
#pragma unroll
            for (int e = 0; e < 8; ++e) ss += f[e] * f[e];
          }
        }
      }
      ss = warp_sum(ss);
      const float inv = rsqrtf(ss / (float)hidden + eps);
      uint4* yr = reinterpret_cast<uint4*>(g + (size_t)row * hidden);
      const uint4* wv = reinterpret_cast<const uint4*>(w);
      for (int v = lane; v < nv; v += 32) {
        float f[8] = {0, 0, 0, 0, 0, 0, 0, 0}, ww[8] = {0, 0, 0, 0, 0, 0, 0, 0}, o[8];
        add8(f, xr[v]);                      // this lane's own store of a moment ago
        add8(ww, wv[v]);
#pragma unroll
        for (int e = 0; e < 8; ++e) o[e] = f[e] * inv * (plus_one ? ww[e] + 1.f : ww[e]);
        const uint4 out = pack8(o);
        if (g_peers == nullptr) {
          yr[v] = out;
        } else {
          // push form of the all-gather: the owner writes its normed row into every rank's g (posted peer stores, a whole
          // 512-byte run per warp instruction); the GEMM that follows only waits for the owners' flags
          for (int p = 0; p < nranks; ++p)
            reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(g_peers[(p + rank) % nranks]) + (size_t)row * hidden)[v] = out;
        }
      }
    }
  }
  // the last CTA to get here closes the call: epoch forward, and (unless something failed) "my rows are final"
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const uint32_t done = atomicAdd(state + 1, 1u);
    if (done == gridDim.x - 1) {
      state[1] = 0;
      state[0] = epoch;
      __threadfence_system();
      const bool bad = err != nullptr && *reinterpret_cast<volatile int*>(err) != 0;
      if (!bad)
        for (int p = 0; p < nranks; ++p)
          st_release_sys(reinterpret_cast<uint32_t*>(flag_peers[p]) + kFlagStride + rank, epoch);
    }
  }
  pdl_launch_dependents();
}

// The last row of every sequence out of the sequence-parallel buffer: row cu_seqlens[i + 1] - 1 lives in its owner's g.
// One CTA per sequence waits (bounded) until that owner's rows are final for this rank's current epoch and copies the
// row over NVLink (or out of local memory when this rank owns it). grid = sequences, block 256.
extern "C" __global__ void __launch_bounds__(kThreads)
    kern_sp_last_rows(const unsigned long long* g_peers, __nv_bfloat16* last, const int* cu_seqlens, const uint32_t* flags,
                      const uint32_t* state, int* err, int rank, int nranks, int seqs, int hidden, long long timeout_ns) {
  __shared__ int failed;
  pdl_wait();
  const int i = blockIdx.x;
  if (i >= seqs) return;
  const int row = cu_seqlens[i + 1] - 1;
  if (row < 0 || cu_seqlens[i + 1] <= cu_seqlens[i]) return;      // a sequence without rows in this call
  const int owner = (row / kSub) % nranks;
  if (threadIdx.x == 0) {
    failed = 0;
    const uint32_t epoch = *reinterpret_cast<const volatile uint32_t*>(state);
    if (owner != rank && !wait_epoch(flags + kFlagStride + owner, epoch, timeout_ns)) {
      set_error(err, ERR_WAIT_PEER + owner);
      failed = 1;
    }
  }
  __syncthreads();
  if (failed) return;
  const uint4* src = reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(g_peers[owner]) + (size_t)row * hidden);
  uint4* dst = reinterpret_cast<uint4*>(last + (size_t)i * hidden);
  for (int v = threadIdx.x; v < hidden / 8; v += kThreads) dst[v] = ld_volatile16(src + v);
  pdl_launch_dependents();
}
