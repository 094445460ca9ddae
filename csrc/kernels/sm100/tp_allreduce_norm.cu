// Tensor-parallel all-reduce over NVLink peer memory fused with the residual add and the RMSNorm that
// follow it in a decoder layer:  x += sum_r partial_r ;  xn = rmsnorm(x) * w  — one kernel, no NCCL.
//
// Every rank launches the same grid; CTA j of every rank owns the same rows (j, j + grid, ...), so the
// only synchronisation is between CTA j of each rank, through per-CTA epoch flags written with
// st.release.sys into the peer's flag array and polled with ld.acquire.sys. Flags carry an epoch kept
// in device memory, so a captured graph replays without host help; staging is double-buffered by epoch
// parity. Every wait is bounded by `timeout_ns` of %globaltimer: a missing rank makes the kernel record
// 200 + rank in *err and return, it never spins forever.
//
//   mode 0 (one-shot, few rows): push my partial rows into my slot on every peer, wait for everyone's,
//          then every rank reduces every row itself in rank order (all ranks produce identical bytes).
//   mode 1 (two-shot, many rows): rows are dealt to owners inside each CTA (row j + i G belongs to rank (i + j) % N); push each partial row to its
//          owner only, the owner reduces (+ residual) and pushes the new x row to every peer, then every
//          rank normalises all of its CTA's rows locally. Link bytes: 2 (N-1)/N of the message.
//   mode 2 (fused with the GEMM): as mode 1, but the partial rows were pushed to their owners by the epilogue of
//          the tensor-parallel GEMM launched just before (tp_gemm.cu); `partial` is not read.
//
// Reference counterpart: tools/kernels-src/peer_allreduce.cu:196-334 (one-shot Lamport and two-shot
// f32 all-reduce; its authors list the fused residual + RMSNorm tail and bf16 partials as not done) and
// tools/kernels-src/peer_barrier.cu:43-58 (bounded flag wait with an error word).
// No cluster multicast anywhere: plain P2P loads/stores only.
#include "common.cuh"

using namespace kern;

namespace {

KERN_DEVICE bool wait_flag(const uint32_t* flag, uint32_t epoch, long long timeout_ns) {
  const uint64_t t0 = globaltimer_ns();
  // epochs wrap after 2^32 calls; compare as a signed distance
  while ((int32_t)(ld_acquire_sys(flag) - epoch) < 0) {
    if ((long long)(globaltimer_ns() - t0) > timeout_ns) return false;
    __nanosleep(20);
  }
  return true;
}

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
// volatile 16-byte load: peer stores must not be served from a stale non-coherent cache line
KERN_DEVICE uint4 ld_volatile16(const void* p) {
  uint4 v;
  asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}

}  // namespace

constexpr int kThreads = 256;

// grid = G CTAs (the same on every rank for a given call, G <= flag_stride), block 256, dyn smem = H*4.
// comm   : [2 parities][nranks slots][slot_rows][H] bf16 on every rank (exported)
// flags  : [2 phases][nranks][flag_stride] u32 on every rank (exported, zero at start); CTA j always uses
//          column j, whatever the grid of the call, so calls of different grids share the epochs
// epochs : [flag_stride] u32 local, zero at start
extern "C" __global__ void __launch_bounds__(kThreads)
    kern_tp_allreduce_residual_norm(const __nv_bfloat16* partial, __nv_bfloat16* x, const unsigned long long* x_peers,
                                    __nv_bfloat16* xn, const __nv_bfloat16* w, __nv_bfloat16* comm,
                                    const unsigned long long* comm_peers, uint32_t* flags,
                                    const unsigned long long* flag_peers, uint32_t* epochs, int* err, int rank, int nranks,
                                    int rows, int hidden, int slot_rows, float eps, int plus_one, int mode,
                                    long long timeout_ns, int flag_stride) {
  extern __shared__ float rowbuf[];   // one row in f32 for the norm
  __shared__ float red[32];
  __shared__ int failed;
  pdl_wait();
  const int j = blockIdx.x, G = gridDim.x;
  const int nv = hidden / 8;
  if (threadIdx.x == 0) failed = 0;
  const uint32_t epoch = epochs[j] + 1;
  __syncthreads();
  if (threadIdx.x == 0) epochs[j] = epoch;
  const int parity = epoch & 1;
  const size_t slot_elems = (size_t)slot_rows * hidden;
  const size_t parity_elems = (size_t)nranks * slot_elems;
  const int my_rows = rows > j ? (rows - j + G - 1) / G : 0;   // rows j, j+G, ... of this CTA

  // ---- phase 1: push partial rows (mode 2: the GEMM before this kernel already did, tile by tile) ----
  for (int i = 0; i < (mode == 2 ? 0 : my_rows); ++i) {
    const int row = j + i * G;
    const uint4* src = reinterpret_cast<const uint4*>(partial + (size_t)row * hidden);
    if (mode == 0) {
      // my slot on every rank (mine included), staging row = row
      if (row >= slot_rows) { if (threadIdx.x == 0) set_error(err, ERR_BOUNDS); continue; }
      for (int p = 0; p < nranks; ++p) {
        __nv_bfloat16* base = reinterpret_cast<__nv_bfloat16*>(comm_peers[p]) + parity * parity_elems + rank * slot_elems;
        uint4* dst = reinterpret_cast<uint4*>(base + (size_t)row * hidden);
        for (int v = threadIdx.x; v < nv; v += kThreads) dst[v] = src[v];
      }
    } else {
      const int owner = (i + j) % nranks;   // rotated by the CTA so a few rows per CTA still spread over every rank
      const int idx = (i / nranks) * G + j;   // dense index among the owner's rows
      if (idx >= slot_rows) { if (threadIdx.x == 0) set_error(err, ERR_BOUNDS); continue; }
      __nv_bfloat16* base = reinterpret_cast<__nv_bfloat16*>(comm_peers[owner]) + parity * parity_elems + rank * slot_elems;
      uint4* dst = reinterpret_cast<uint4*>(base + (size_t)idx * hidden);
      for (int v = threadIdx.x; v < nv; v += kThreads) dst[v] = src[v];
    }
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x < nranks)
    st_release_sys(reinterpret_cast<uint32_t*>(flag_peers[threadIdx.x]) + (size_t)(0 * nranks + rank) * flag_stride + j, epoch);
  if (threadIdx.x < nranks) {
    if (!wait_flag(flags + (size_t)(0 * nranks + threadIdx.x) * flag_stride + j, epoch, timeout_ns)) {
      set_error(err, ERR_WAIT_PEER + threadIdx.x);
      failed = 1;
    }
  }
  __syncthreads();

  const __nv_bfloat16* mine = comm + parity * parity_elems;
  // ---- phase 2: reduce (+ residual) ----
  if (!failed) {
    for (int i = 0; i < my_rows; ++i) {
      const int row = j + i * G;
      int idx = row;
      if (mode >= 1) {
        if ((i + j) % nranks != rank) continue;   // not my row to reduce
        idx = (i / nranks) * G + j;
      }
      if (idx >= slot_rows) continue;
      uint4* xr = reinterpret_cast<uint4*>(x + (size_t)row * hidden);
      for (int v = threadIdx.x; v < nv; v += kThreads) {
        float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        for (int r = 0; r < nranks; ++r)   // rank order: every rank adds in the same order
          add8(acc, ld_volatile16(reinterpret_cast<const uint4*>(mine + r * slot_elems + (size_t)idx * hidden) + v));
        // partial sums are rounded to bf16 once, then the residual is added as the unfused epilogue would
        uint4 s = pack8(acc);
        float tot[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        add8(tot, s);
        add8(tot, xr[v]);
        const uint4 out = pack8(tot);
        if (mode == 0) {
          xr[v] = out;
        } else {
          for (int p = 0; p < nranks; ++p)
            reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(x_peers[p]) + (size_t)row * hidden)[v] = out;
        }
      }
    }
  }
  if (mode >= 1) {
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x < nranks)
      st_release_sys(reinterpret_cast<uint32_t*>(flag_peers[threadIdx.x]) + (size_t)(1 * nranks + rank) * flag_stride + j, epoch);
    if (threadIdx.x < nranks && !failed) {
      if (!wait_flag(flags + (size_t)(1 * nranks + threadIdx.x) * flag_stride + j, epoch, timeout_ns)) {
        set_error(err, ERR_WAIT_PEER + threadIdx.x);
        failed = 1;
      }
    }
  }
  __syncthreads();
  if (failed) return;

  // ---- phase 3: RMSNorm of every row of this CTA ----
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int i = 0; i < my_rows; ++i) {
    const int row = j + i * G;
    const uint4* xr = reinterpret_cast<const uint4*>(x + (size_t)row * hidden);
    float ss = 0.f;
    for (int v = threadIdx.x; v < nv; v += kThreads) {
      float f[8] = {0, 0, 0, 0, 0, 0, 0, 0};
      add8(f, mode >= 1 ? ld_volatile16(xr + v) : xr[v]);
#pragma unroll
      for (int e = 0; e < 8; ++e) { rowbuf[v * 8 + e] = f[e]; ss += f[e] * f[e]; }
    }
    ss = warp_sum(ss);
    if (lane == 0) red[warp] = ss;
    __syncthreads();
    if (warp == 0) {
      float t = lane < kThreads / 32 ? red[lane] : 0.f;
      t = warp_sum(t);
      if (lane == 0) red[0] = t;
    }
    __syncthreads();
    const float inv = rsqrtf(red[0] / (float)hidden + eps);
    uint4* yr = reinterpret_cast<uint4*>(xn + (size_t)row * hidden);
    const uint4* wv = reinterpret_cast<const uint4*>(w);
    for (int v = threadIdx.x; v < nv; v += kThreads) {
      float ww[8] = {0, 0, 0, 0, 0, 0, 0, 0}, o[8];
      add8(ww, wv[v]);
#pragma unroll
      for (int e = 0; e < 8; ++e) o[e] = rowbuf[v * 8 + e] * inv * (plus_one ? ww[e] + 1.f : ww[e]);
      yr[v] = pack8(o);
    }
    __syncthreads();
  }
  pdl_launch_dependents();
}

// Cross-rank barrier with a bounded wait: every rank writes the next epoch into its flag word on every
// peer and waits for all of theirs. err = 200 + first missing rank on timeout. grid 1, block 32.
// Reference counterpart: tools/kernels-src/peer_barrier.cu:32.
extern "C" __global__ void kern_peer_barrier(uint32_t* flags, const unsigned long long* flag_peers, uint32_t* epoch_word,
                                             int* err, int rank, int nranks, long long timeout_ns) {
  pdl_wait();
  const uint32_t epoch = epoch_word[0] + 1;
  __syncwarp();
  if (threadIdx.x == 0) epoch_word[0] = epoch;
  __threadfence_system();
  if ((int)threadIdx.x < nranks) {
    st_release_sys(reinterpret_cast<uint32_t*>(flag_peers[threadIdx.x]) + rank, epoch);
    if (!wait_flag(flags + threadIdx.x, epoch, timeout_ns)) set_error(err, ERR_WAIT_PEER + threadIdx.x);
  }
}

// ---- one-shot all-reduce without flags (few rows: decode steps) ------------------------------------------------
// The payload is its own arrival signal: every 16-bit word of a staging buffer starts as the poison 0x8000 (bf16 -0.0),
// senders never store that value (a partial that is exactly -0.0 travels as +0.0, the same number), so a receiver just
// polls the vector it needs until none of its eight words is poison. No flag write, no second round trip.
// Three staging buffers rotate by the CTA's epoch: a call writes stage e % 3, reads it, and re-poisons its rows of
// stage (e + 2) % 3 — the one the previous call used, which no peer writes again before it has consumed this call's
// rows. grid = rows (CTA j owns row j, on every rank), block 256, dyn smem = hidden * 4.
//   lamport : [3 stages][nranks slots][slot_rows][hidden] bf16 on every rank (exported, poisoned by a `once` fill)
// Reference counterpart: tools/kernels-src/peer_allreduce.cu:196-259 (f32 payload, -0.0 poison, three stages).
namespace {
constexpr uint32_t kPoison2 = 0x80008000u;
KERN_DEVICE bool has_poison(uint4 v) {
  auto p = [](uint32_t w) { return (w & 0xffffu) == 0x8000u || (w >> 16) == 0x8000u; };
  return p(v.x) || p(v.y) || p(v.z) || p(v.w);
}
KERN_DEVICE uint32_t scrub2(uint32_t w) {   // -0.0 -> +0.0 in either half
  if ((w & 0xffffu) == 0x8000u) w &= 0xffff0000u;
  if ((w >> 16) == 0x8000u) w &= 0x0000ffffu;
  return w;
}
}  // namespace

extern "C" __global__ void __launch_bounds__(kThreads)
    kern_tp_allreduce_lamport(const __nv_bfloat16* partial, __nv_bfloat16* x, __nv_bfloat16* xn, const __nv_bfloat16* w,
                              __nv_bfloat16* lamport, const unsigned long long* lamport_peers, uint32_t* epochs, int* err,
                              int rank, int nranks, int rows, int hidden, int slot_rows, float eps, int plus_one,
                              long long timeout_ns) {
  extern __shared__ float rowbuf[];
  __shared__ float red[32];
  __shared__ int failed;
  pdl_wait();
  const int row = blockIdx.x;
  if (row >= rows) return;
  if (row >= slot_rows) { if (threadIdx.x == 0) set_error(err, ERR_BOUNDS); return; }
  const int nv = hidden / 8;
  if (threadIdx.x == 0) failed = 0;
  const uint32_t epoch = epochs[row] + 1;
  __syncthreads();
  if (threadIdx.x == 0) epochs[row] = epoch;
  const size_t slot_elems = (size_t)slot_rows * hidden;
  const size_t stage_elems = (size_t)nranks * slot_elems;
  const uint32_t stage = epoch % 3, clear = (epoch + 2) % 3;

  // push my row into my slot of this stage on every rank (mine included)
  const uint4* src = reinterpret_cast<const uint4*>(partial + (size_t)row * hidden);
  for (int v = threadIdx.x; v < nv; v += kThreads) {
    uint4 d = src[v];
    d.x = scrub2(d.x); d.y = scrub2(d.y); d.z = scrub2(d.z); d.w = scrub2(d.w);
    for (int p = 0; p < nranks; ++p) {
      __nv_bfloat16* base = reinterpret_cast<__nv_bfloat16*>(lamport_peers[p]) + stage * stage_elems + rank * slot_elems;
      reinterpret_cast<uint4*>(base + (size_t)row * hidden)[v] = d;
    }
  }
  // re-poison my row of the stage used two calls from now
  for (int r = 0; r < nranks; ++r) {
    uint4* c = reinterpret_cast<uint4*>(lamport + clear * stage_elems + r * slot_elems + (size_t)row * hidden);
    for (int v = threadIdx.x; v < nv; v += kThreads) c[v] = make_uint4(kPoison2, kPoison2, kPoison2, kPoison2);
  }
  // gather: poll each rank's vector until it is whole, sum in rank order, add the residual
  const __nv_bfloat16* mine = lamport + stage * stage_elems;
  uint4* xr = reinterpret_cast<uint4*>(x + (size_t)row * hidden);
  float ss = 0.f;
  const uint64_t t0 = globaltimer_ns();
  for (int v = threadIdx.x; v < nv; v += kThreads) {
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    bool ok = true;
    for (int r = 0; r < nranks && ok; ++r) {
      const uint4* p = reinterpret_cast<const uint4*>(mine + r * slot_elems + (size_t)row * hidden) + v;
      uint4 d = ld_volatile16(p);
      while (has_poison(d)) {
        if ((long long)(globaltimer_ns() - t0) > timeout_ns) {
          set_error(err, ERR_WAIT_PEER + r);
          failed = 1;
          ok = false;
          break;
        }
        d = ld_volatile16(p);
      }
      if (ok) add8(acc, d);
    }
    if (!ok) break;
    uint4 s = pack8(acc);
    float tot[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    add8(tot, s);
    add8(tot, xr[v]);
    const uint4 out = pack8(tot);
    xr[v] = out;
    float f[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    add8(f, out);
#pragma unroll
    for (int e = 0; e < 8; ++e) { rowbuf[v * 8 + e] = f[e]; ss += f[e] * f[e]; }
  }
  __syncthreads();
  if (failed) return;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  ss = warp_sum(ss);
  if (lane == 0) red[warp] = ss;
  __syncthreads();
  if (warp == 0) {
    float t = lane < kThreads / 32 ? red[lane] : 0.f;
    t = warp_sum(t);
    if (lane == 0) red[0] = t;
  }
  __syncthreads();
  const float inv = rsqrtf(red[0] / (float)hidden + eps);
  uint4* yr = reinterpret_cast<uint4*>(xn + (size_t)row * hidden);
  const uint4* wv = reinterpret_cast<const uint4*>(w);
  for (int v = threadIdx.x; v < nv; v += kThreads) {
    float ww[8] = {0, 0, 0, 0, 0, 0, 0, 0}, o[8];
    add8(ww, wv[v]);
#pragma unroll
    for (int e = 0; e < 8; ++e) o[e] = rowbuf[v * 8 + e] * inv * (plus_one ? ww[e] + 1.f : ww[e]);
    yr[v] = pack8(o);
  }
  pdl_launch_dependents();
}

// ---- all-gather over peer memory -------------------------------------------------------------------------------
// Every rank contributes `bytes` bytes (a multiple of 16); afterwards y on every rank holds the nranks blocks in rank
// order. Each CTA j moves its slice of the local block into slot [parity][rank] of every peer's staging buffer, raises
// its epoch flag on every peer, waits (bounded) for every peer's flag of the same CTA, then copies its slice of all
// slots out to y. Parity double-buffering lets the next call start while a slow peer still reads this one.
//   sym   : [2 parities][nranks][slot_bytes] on every rank (exported);   flags: [nranks][flag_stride] u32 (exported)
// grid G <= flag_stride (the same on every rank), block 256.
// Reference counterpart: tools/kernels-src/peer_collective.cu:128 (LL-style all-gather with per-CTA epochs).
extern "C" __global__ void __launch_bounds__(kThreads)
    kern_peer_allgather(const uint8_t* x, uint8_t* y, uint8_t* sym, const unsigned long long* sym_peers, uint32_t* flags,
                        const unsigned long long* flag_peers, uint32_t* epochs, int* err, int rank, int nranks,
                        long long bytes, long long slot_bytes, long long timeout_ns, int flag_stride) {
  __shared__ int failed;
  pdl_wait();
  const int j = blockIdx.x, G = gridDim.x;
  if (threadIdx.x == 0) failed = 0;
  const uint32_t epoch = epochs[j] + 1;
  __syncthreads();
  if (threadIdx.x == 0) epochs[j] = epoch;
  if (bytes > slot_bytes || (bytes & 15)) {
    if (threadIdx.x == 0) set_error(err, ERR_BOUNDS);
    return;
  }
  const long long parity_off = (long long)(epoch & 1) * nranks * slot_bytes;
  const long long nvec = bytes / 16;
  const long long per = (nvec + G - 1) / G, lo = j * per, hi = lo + per < nvec ? lo + per : nvec;
  const uint4* src = reinterpret_cast<const uint4*>(x);
  for (int p = 0; p < nranks; ++p) {
    uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<uint8_t*>(sym_peers[p]) + parity_off + (long long)rank * slot_bytes);
    for (long long v = lo + threadIdx.x; v < hi; v += kThreads) dst[v] = src[v];
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x < nranks) {
    st_release_sys(reinterpret_cast<uint32_t*>(flag_peers[threadIdx.x]) + (size_t)rank * flag_stride + j, epoch);
    if (!wait_flag(flags + (size_t)threadIdx.x * flag_stride + j, epoch, timeout_ns)) {
      set_error(err, ERR_WAIT_PEER + threadIdx.x);
      failed = 1;
    }
  }
  __syncthreads();
  if (failed) return;
  for (int r = 0; r < nranks; ++r) {
    const uint4* s = reinterpret_cast<const uint4*>(sym + parity_off + (long long)r * slot_bytes);
    uint4* d = reinterpret_cast<uint4*>(y + (long long)r * bytes);
    for (long long v = lo + threadIdx.x; v < hi; v += kThreads) d[v] = ld_volatile16(s + v);
  }
  pdl_launch_dependents();
}
