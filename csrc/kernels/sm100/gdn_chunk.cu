// Gated delta rule for prefill chunks in its chunked (WY) form: the token-by-token recurrence of gdn.cu issues about
// 118 instructions per token per warp and cannot go faster than that; here 64 tokens at a time become small matrix
// products on the tensor cores, and only the state-dependent part stays sequential (one step per 64 tokens).
//
// Per chunk of 64 tokens of one (sequence, value head), with g the inclusive cumulative log decay inside the chunk:
//   L[i,j] = beta_i exp(g_i - g_j) (k_i.k_j), j < i          T = (I + L)^-1   (unit lower triangular)
//   W = T (beta exp(g) K)      Ut = T (beta V)      Qg = exp(g) q      Kd = exp(g_last - g) k
//   M[i,j] = exp(g_i - g_j) (q_i.k_j), j <= i                gC = exp(g_last)
// and with S0 the state entering the chunk:
//   U = Ut - W S0^T        O = Qg S0^T + M U        S1 = gC S0 + U^T Kd
//
//   kern_gdn_chunk_prep_k128_v128   everything above the last line: parallel over (chunk, head); writes W, Qg, Kd, Ut, M,
//                                   gC to scratch, already rounded to tf32 (the format the second kernel multiplies in)
//   kern_gdn_chunk_rule_k128_v128   the last line: a CTA per (sequence, head, half of the value rows) walks the chunks
//                                   with the state in registers (as accumulator fragments) and in shared memory (as an
//                                   operand); cp.async refills each operand buffer as soon as its product is done
//
// The products are tf32 mma.sync (m16n8k8, f32 accumulate): the tiles are 64 x 64 x 128 at most, too small and too
// dependent on one another for a TMEM pipeline to pay, and tf32 keeps three more mantissa bits than bf16 operands would.
// The reference takes this kernel from a mined Triton build (chunked GDN prefill); it has no source there.
#include "common.cuh"

using namespace kern;

namespace {

constexpr int CH = 64;        // tokens per chunk
constexpr int DD = 128;       // DK = DV
constexpr int LDK = DD + 4;   // row stride (floats) of operand tiles read as A[m][k] or as B[k][n] = X[n][k]: bank 4 g + t
constexpr int LDN = DD + 8;   // row stride of tiles read as B[k][n] = X[k][n]: bank 8 t + g
constexpr int LDL = CH + 4;   // 64 x 64 tiles read as A
constexpr int LDU = CH + 8;   // 64 x 64 tiles read as B[k][n] = X[k][n] and as A[m][k] = X[k][m]

KERN_DEVICE float tf32r(float x) {
  uint32_t r;
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(x));
  return __uint_as_float(r);
}

KERN_DEVICE void mma_tf32(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// acc[nt] (16 x 8 each, columns 8 nt ..) += A[16 x 8 ksteps] . B[8 ksteps x 8 NT]; a_at(m, k), b_at(k, n) return the
// operand element as f32 bits (already tf32-rounded where it matters).
template <int NT, class FA, class FB>
KERN_DEVICE void warp_mma(float (&acc)[NT][4], int ksteps, FA a_at, FB b_at) {
  const int lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  for (int ks = 0; ks < ksteps; ++ks) {
    const int k0 = ks * 8;
    const uint32_t a[4] = {a_at(g, k0 + t), a_at(g + 8, k0 + t), a_at(g, k0 + t + 4), a_at(g + 8, k0 + t + 4)};
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) mma_tf32(acc[nt], a, b_at(k0 + t, nt * 8 + g), b_at(k0 + t + 4, nt * 8 + g));
  }
}

KERN_DEVICE void cp_async16(void* dst, const void* src, bool valid) {
  const uint32_t bytes = valid ? 16u : 0u;     // 0: nothing is read, the 16 bytes are filled with zeros
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_u32(dst)), "l"(src), "r"(bytes) : "memory");
}
KERN_DEVICE void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
KERN_DEVICE void cp_async_wait_all() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }

// Which (sequence, chunk) a chunk slot of the grid is: sequences are walked in order, each owns ceil(rows / 64) slots.
KERN_DEVICE bool chunk_of(const int* cu_q, int seqs, int slot, int& r0, int& nvalid) {
  for (int s = 0; s < seqs; ++s) {
    const int a = cu_q[s], b = cu_q[s + 1];
    const int nc = (b - a + CH - 1) / CH;
    if (slot < nc) {
      r0 = a + slot * CH;
      nvalid = min(CH, b - r0);
      return true;
    }
    slot -= nc;
  }
  return false;
}

}  // namespace

// T = (I + L)^-1, then W = T Ks and Ut = T Qs to scratch (Ks holds beta-scaled decayed keys, Qs beta v); shared by
// the scalar-decay and the per-key-decay preparation.
KERN_DEVICE void solve_and_project(float (*Ls)[LDL], float (*Ks)[LDK], float (*Qs)[LDK], float* Wg, float* Ug, int r0,
                                   int nvalid, int hv, int h) {
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t4 = lane & 3;
  // T = (I + L)^-1 by forward substitution: thread j owns column j (row t needs rows < t of the same column only);
  // the row of L is a broadcast read, two accumulators halve the dependent chain
  float Tc[CH];
  if (tid < CH) {
#pragma unroll
    for (int t = 0; t < CH; ++t) {
      float a0 = t == tid ? 1.f : 0.f, a1 = 0.f;
#pragma unroll
      for (int i4 = 0; i4 < t / 4; ++i4) {
        const float4 l = *reinterpret_cast<const float4*>(&Ls[t][4 * i4]);
        a0 -= l.x * Tc[4 * i4];
        a1 -= l.y * Tc[4 * i4 + 1];
        a0 -= l.z * Tc[4 * i4 + 2];
        a1 -= l.w * Tc[4 * i4 + 3];
      }
#pragma unroll
      for (int i = (t / 4) * 4; i < t; ++i) a0 -= Ls[t][i] * Tc[i];
      Tc[t] = a0 + a1;
    }
  }
  __syncthreads();      // every column is done reading L
  if (tid < CH) {
#pragma unroll
    for (int t = 0; t < CH; ++t) Ls[t][tid] = tf32r(Tc[t]);
  }
  __syncthreads();

  // W = T (beta exp(g) K), Ut = T (beta V): warp -> rows 16 mb .., columns 64 nh ..; T is lower triangular, so the
  // products stop at the diagonal block
  {
    const int mb = warp & 3, nh = warp >> 2;
    float w[8][4], u[8][4];
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) { w[i][j] = 0.f; u[i][j] = 0.f; }
    auto a_at = [&](int m, int k) { return __float_as_uint(Ls[16 * mb + m][k]); };
    warp_mma<8>(w, 2 * (mb + 1), a_at, [&](int k, int n) { return __float_as_uint(Ks[k][64 * nh + n]); });
    warp_mma<8>(u, 2 * (mb + 1), a_at, [&](int k, int n) { return __float_as_uint(Qs[k][64 * nh + n]); });
#pragma unroll
    for (int nt = 0; nt < 8; ++nt)
#pragma unroll
      for (int hh = 0; hh < 2; ++hh) {
        const int i = 16 * mb + g + 8 * hh, col = 64 * nh + 8 * nt + 2 * t4;
        if (i < nvalid) {
          const size_t at = ((size_t)(r0 + i) * hv + h) * DD + col;
          *reinterpret_cast<float2*>(Wg + at) = make_float2(tf32r(w[nt][2 * hh]), tf32r(w[nt][2 * hh + 1]));
          *reinterpret_cast<float2*>(Ug + at) = make_float2(tf32r(u[nt][2 * hh]), tf32r(u[nt][2 * hh + 1]));
        }
      }
  }
}

// grid [ceil(tokens / 64) + seqs, HV], block 256, dynamic shared memory PREP_SMEM bytes.
// Scratch: W, Qg, Kd, Ut [tokens, HV, 128] f32; M [tokens, HV, 64] f32; gC [tokens, HV] f32.
constexpr int PREP_SMEM = (2 * CH * LDK + CH * LDL + 2 * CH) * 4;

extern "C" __global__ void __launch_bounds__(256, 2)
    kern_gdn_chunk_prep_k128_v128(const __nv_bfloat16* qkv, const __nv_bfloat16* zba, const int* cu_q, const float* A_log,
                                  const float* dt_bias, float* Wg, float* Qg, float* Kg, float* Ug, float* Mg, float* Gg,
                                  int seqs, int hk, int hv, int zba_stride, int b_off, int a_off) {
  pdl_wait();
  extern __shared__ __align__(16) float sm[];
  float (*Ks)[LDK] = reinterpret_cast<float (*)[LDK]>(sm);                    // k, later beta exp(g) k
  float (*Qs)[LDK] = reinterpret_cast<float (*)[LDK]>(sm + CH * LDK);         // q, later beta v
  float (*Ls)[LDL] = reinterpret_cast<float (*)[LDL]>(sm + 2 * CH * LDK);     // L, later T
  float* gs = sm + 2 * CH * LDK + CH * LDL;                                   // log decay, then its running sum
  float* bs = gs + CH;                                                        // beta
  int r0, nvalid;
  if (!chunk_of(cu_q, seqs, blockIdx.x, r0, nvalid)) return;
  const int h = blockIdx.y, kh = h / (hv / hk);
  const int conv_dim = 2 * hk * DD + hv * DD;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t4 = lane & 3;

  // v: 8 x 16-byte pieces... issued first so the loads fly under the normalisation; piece p = (token, 8 columns)
  uint4 vreg[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int p = tid + 256 * i, tok = p >> 4, c8 = p & 15;
    vreg[i] = tok < nvalid ? *reinterpret_cast<const uint4*>(qkv + (size_t)(r0 + tok) * conv_dim + 2 * hk * DD + h * DD + c8 * 8)
                           : make_uint4(0u, 0u, 0u, 0u);
  }
  // q, k: a warp takes tokens warp, warp + 8, ...; a lane holds 4 consecutive columns of each
  {
    const float a_neg = -__expf(A_log[h]);
    const float dtb = dt_bias[h];
    uint2 rq[8], rk[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const int tok = warp + 8 * u;
      const __nv_bfloat16* row = qkv + (size_t)(r0 + tok) * conv_dim;
      rq[u] = tok < nvalid ? *reinterpret_cast<const uint2*>(row + kh * DD + lane * 4) : make_uint2(0u, 0u);
      rk[u] = tok < nvalid ? *reinterpret_cast<const uint2*>(row + hk * DD + kh * DD + lane * 4) : make_uint2(0u, 0u);
    }
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const int tok = warp + 8 * u;
      const float2 q01 = unpack_bf16x2(rq[u].x), q23 = unpack_bf16x2(rq[u].y);
      const float2 k01 = unpack_bf16x2(rk[u].x), k23 = unpack_bf16x2(rk[u].y);
      float q2 = q01.x * q01.x + q01.y * q01.y + q23.x * q23.x + q23.y * q23.y;
      float k2 = k01.x * k01.x + k01.y * k01.y + k23.x * k23.x + k23.y * k23.y;
      q2 = warp_sum(q2);
      k2 = warp_sum(k2);
      const float qi = rsqrtf(q2 + 1e-6f) * rsqrtf((float)DD), ki = rsqrtf(k2 + 1e-6f);
      *reinterpret_cast<float4*>(&Qs[tok][lane * 4]) =
          make_float4(tf32r(q01.x * qi), tf32r(q01.y * qi), tf32r(q23.x * qi), tf32r(q23.y * qi));
      *reinterpret_cast<float4*>(&Ks[tok][lane * 4]) =
          make_float4(tf32r(k01.x * ki), tf32r(k01.y * ki), tf32r(k23.x * ki), tf32r(k23.y * ki));
      if (lane == 0) {
        float ga = 0.f, be = 0.f;
        if (tok < nvalid) {
          const float av = __bfloat162float(zba[(size_t)(r0 + tok) * zba_stride + a_off + h]) + dtb;
          const float sp = av > 20.f ? av : log1pf(__expf(av));
          const float bb = __bfloat162float(zba[(size_t)(r0 + tok) * zba_stride + b_off + h]);
          ga = a_neg * sp;
          be = __bfloat162float(__float2bfloat16(1.f / (1.f + __expf(-bb))));
        }
        gs[tok] = ga;
        bs[tok] = be;
      }
    }
  }
  __syncthreads();
  if (warp == 0) {      // inclusive running sum of the log decays over the 64 tokens (padding rows add 0)
    float x0 = gs[lane], x1 = gs[lane + 32];
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const float y0 = __shfl_up_sync(0xffffffffu, x0, o), y1 = __shfl_up_sync(0xffffffffu, x1, o);
      if (lane >= o) { x0 += y0; x1 += y1; }
    }
    x1 += __shfl_sync(0xffffffffu, x0, 31);
    gs[lane] = x0;
    gs[lane + 32] = x1;
  }
  __syncthreads();
  const float g_last = gs[CH - 1];

  // k.k and q.k over the chunk: warp -> rows 16 mb .., columns 32 nh ..; blocks above the diagonal are skipped
  {
    const int mb = warp & 3, nh = warp >> 2;
    if (32 * nh <= 16 * mb + 15) {
      float kk[4][4], qk[4][4];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) { kk[i][j] = 0.f; qk[i][j] = 0.f; }
      auto b_at = [&](int k, int n) { return __float_as_uint(Ks[32 * nh + n][k]); };
      warp_mma<4>(kk, DD / 8, [&](int m, int k) { return __float_as_uint(Ks[16 * mb + m][k]); }, b_at);
      warp_mma<4>(qk, DD / 8, [&](int m, int k) { return __float_as_uint(Qs[16 * mb + m][k]); }, b_at);
#pragma unroll
      for (int nt = 0; nt < 4; ++nt)
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
          const int i = 16 * mb + g + 8 * hh, j = 32 * nh + 8 * nt + 2 * t4;
          const float gi = gs[i], bi = bs[i];
          const float e0 = j <= i ? __expf(gi - gs[j]) : 0.f, e1 = j + 1 <= i ? __expf(gi - gs[j + 1]) : 0.f;
          Ls[i][j] = j < i ? bi * e0 * kk[nt][2 * hh] : 0.f;
          Ls[i][j + 1] = j + 1 < i ? bi * e1 * kk[nt][2 * hh + 1] : 0.f;
          if (i < nvalid)
            *reinterpret_cast<float2*>(Mg + ((size_t)(r0 + i) * hv + h) * CH + j) =
                make_float2(tf32r(e0 * qk[nt][2 * hh]), tf32r(e1 * qk[nt][2 * hh + 1]));
        }
    } else {
      // the skipped block is all zeros in L and M
#pragma unroll
      for (int nt = 0; nt < 4; ++nt)
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
          const int i = 16 * mb + g + 8 * hh, j = 32 * nh + 8 * nt + 2 * t4;
          Ls[i][j] = 0.f;
          Ls[i][j + 1] = 0.f;
          if (i < nvalid) *reinterpret_cast<float2*>(Mg + ((size_t)(r0 + i) * hv + h) * CH + j) = make_float2(0.f, 0.f);
        }
    }
  }
  __syncthreads();      // L complete; nobody reads raw q or k through the tensor path any more

  // Qg and Kd leave for scratch; k becomes beta exp(g) k in place and beta v takes q's place (a thread rewrites only
  // the elements it has just read)
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int p = tid + 256 * i, tok = p >> 4, c0 = (p & 15) * 8;
    const float eg = __expf(gs[tok]), ed = __expf(g_last - gs[tok]), be = bs[tok];
    const float2 v01 = unpack_bf16x2(vreg[i].x), v23 = unpack_bf16x2(vreg[i].y), v45 = unpack_bf16x2(vreg[i].z),
                 v67 = unpack_bf16x2(vreg[i].w);
    const float vv[8] = {v01.x, v01.y, v23.x, v23.y, v45.x, v45.y, v67.x, v67.y};
    float qo[8], ko[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const float q = Qs[tok][c0 + e], k = Ks[tok][c0 + e];
      qo[e] = tf32r(eg * q);
      ko[e] = tf32r(ed * k);
      Ks[tok][c0 + e] = tf32r(be * eg * k);
      Qs[tok][c0 + e] = tf32r(be * vv[e]);
    }
    if (tok < nvalid) {
      float* qd = Qg + ((size_t)(r0 + tok) * hv + h) * DD + c0;
      float* kd = Kg + ((size_t)(r0 + tok) * hv + h) * DD + c0;
      *reinterpret_cast<float4*>(qd) = make_float4(qo[0], qo[1], qo[2], qo[3]);
      *reinterpret_cast<float4*>(qd + 4) = make_float4(qo[4], qo[5], qo[6], qo[7]);
      *reinterpret_cast<float4*>(kd) = make_float4(ko[0], ko[1], ko[2], ko[3]);
      *reinterpret_cast<float4*>(kd + 4) = make_float4(ko[4], ko[5], ko[6], ko[7]);
    }
  }
  if (tid < nvalid) Gg[(size_t)(r0 + tid) * hv + h] = __expf(g_last);

  solve_and_project(Ls, Ks, Qs, Wg, Ug, r0, nvalid, hv, h);
}

// ---- per-key decay (Kimi Delta Attention) ---------------------------------------------------------------------------
// The same factors with g a vector over the keys: G[t][k] the inclusive running sum of log2 decay inside the chunk.
//   L[i,j] = beta_i sum_k k_i[k] k_j[k] 2^(G_i[k] - G_j[k])  (j < i)      M[i,j] = sum_k q_i[k] k_j[k] 2^(G_i[k] - G_j[k])  (j <= i)
//   W = T (beta 2^G K)     Qg = 2^G q     Kd = 2^(G_last - G) k     Dg = 2^G_last (a vector)
// The pairwise sums are not matrix products (the weight depends on i, j and k), and k / 2^G overflows under strong
// decay, so they run on the CUDA cores with every exponent <= 0: tokens fall in four groups of 16; for j in an earlier
// group than i,   2^(G_i - G_j) = 2^(G_i - R_a) . 2^(R_a - R_b') . 2^(R_b' - G_j)
// (R_a: the sum just before group a of i; R_b': the sum at the end of j's group) — the last factor is folded into the
// keys as they are loaded, the middle one is a 3-row table, the first costs one exp2 per (i, k); pairs inside a
// group take 2^(G_i - G_j) directly. A thread owns rows {bi + 16 a} x columns {bj + 16 b}: ten live pairs each.
// grid [ceil(tokens / 64) + seqs, HV], block 256, dynamic shared memory KDA_PREP_SMEM bytes.
constexpr int KDA_PREP_SMEM = (3 * CH * LDK + CH + 3 * DD) * 4;      // 103 KB: two CTAs per SM

extern "C" __global__ void __launch_bounds__(256, 2)
    kern_kda_chunk_prep_k128_v128(const __nv_bfloat16* qkv, const __nv_bfloat16* zba, const __nv_bfloat16* gk, const int* cu_q,
                                  const float* A_log, const float* dt_bias, float* Wg, float* Qg, float* Kg, float* Ug,
                                  float* Mg, float* Dg, int seqs, int hk, int hv, int zba_stride, int b_off, int gk_stride) {
  pdl_wait();
  extern __shared__ __align__(16) float sm[];
  float (*Ks)[LDK] = reinterpret_cast<float (*)[LDK]>(sm);                    // k, later beta 2^G k
  float (*Qs)[LDK] = reinterpret_cast<float (*)[LDK]>(sm + CH * LDK);         // q, later beta v
  float (*Gs)[LDK] = reinterpret_cast<float (*)[LDK]>(sm + 2 * CH * LDK);     // log2 decay, then its running sum
  float (*Ls)[LDL] = reinterpret_cast<float (*)[LDL]>(sm + 2 * CH * LDK);     // L, later T: over Gs, once Gs has been used
  float* bs = sm + 3 * CH * LDK;                                              // beta
  float (*Dt)[DD] = reinterpret_cast<float (*)[DD]>(bs + CH);                 // 2^(R_2 - R_1), 2^(R_3 - R_1), 2^(R_3 - R_2)
  int r0, nvalid;
  if (!chunk_of(cu_q, seqs, blockIdx.x, r0, nvalid)) return;
  const int h = blockIdx.y, kh = h / (hv / hk);
  const int conv_dim = 2 * hk * DD + hv * DD;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

  uint4 vreg[4];
  {
    const float a2 = -__expf(A_log[h]) * 1.4426950408889634f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int p = tid + 256 * i, tok = p >> 4, c8 = p & 15;
      const bool ok = tok < nvalid;
      vreg[i] = ok ? *reinterpret_cast<const uint4*>(qkv + (size_t)(r0 + tok) * conv_dim + 2 * hk * DD + h * DD + c8 * 8)
                   : make_uint4(0u, 0u, 0u, 0u);
      const uint4 gr = ok ? *reinterpret_cast<const uint4*>(gk + (size_t)(r0 + tok) * gk_stride + h * DD + c8 * 8)
                          : make_uint4(0u, 0u, 0u, 0u);
      const float2 g01 = unpack_bf16x2(gr.x), g23 = unpack_bf16x2(gr.y), g45 = unpack_bf16x2(gr.z), g67 = unpack_bf16x2(gr.w);
      const float gv[8] = {g01.x, g01.y, g23.x, g23.y, g45.x, g45.y, g67.x, g67.y};
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const float x = gv[e] + dt_bias[h * DD + c8 * 8 + e];
        Gs[tok][c8 * 8 + e] = ok ? a2 * (x > 20.f ? x : log1pf(__expf(x))) : 0.f;      // padding rows decay nothing
      }
    }
    uint2 rq[8], rk[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const int tok = warp + 8 * u;
      const __nv_bfloat16* row = qkv + (size_t)(r0 + tok) * conv_dim;
      rq[u] = tok < nvalid ? *reinterpret_cast<const uint2*>(row + kh * DD + lane * 4) : make_uint2(0u, 0u);
      rk[u] = tok < nvalid ? *reinterpret_cast<const uint2*>(row + hk * DD + kh * DD + lane * 4) : make_uint2(0u, 0u);
    }
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const int tok = warp + 8 * u;
      const float2 q01 = unpack_bf16x2(rq[u].x), q23 = unpack_bf16x2(rq[u].y);
      const float2 k01 = unpack_bf16x2(rk[u].x), k23 = unpack_bf16x2(rk[u].y);
      float q2 = q01.x * q01.x + q01.y * q01.y + q23.x * q23.x + q23.y * q23.y;
      float k2 = k01.x * k01.x + k01.y * k01.y + k23.x * k23.x + k23.y * k23.y;
      q2 = warp_sum(q2);
      k2 = warp_sum(k2);
      const float qi = rsqrtf(q2 + 1e-6f) * rsqrtf((float)DD), ki = rsqrtf(k2 + 1e-6f);
      *reinterpret_cast<float4*>(&Qs[tok][lane * 4]) = make_float4(q01.x * qi, q01.y * qi, q23.x * qi, q23.y * qi);
      *reinterpret_cast<float4*>(&Ks[tok][lane * 4]) = make_float4(k01.x * ki, k01.y * ki, k23.x * ki, k23.y * ki);
      if (lane == 0) {
        float be = 0.f;
        if (tok < nvalid) {
          const float bb = __bfloat162float(zba[(size_t)(r0 + tok) * zba_stride + b_off + h]);
          be = __bfloat162float(__float2bfloat16(1.f / (1.f + __expf(-bb))));
        }
        bs[tok] = be;
      }
    }
  }
  __syncthreads();
  if (tid < DD) {      // running sum over the 64 tokens, one key column per thread
    float run = 0.f;
#pragma unroll 8
    for (int t = 0; t < CH; ++t) {
      run += Gs[t][tid];
      Gs[t][tid] = run;
    }
  }
  __syncthreads();
  // the group-to-group table
  for (int p = tid; p < 3 * DD; p += 256) {
    const int which = p / DD, k = p % DD;
    const int hi = which == 0 ? 31 : 47, lo = which == 2 ? 31 : 15;      // R_2 - R_1, R_3 - R_1, R_3 - R_2
    Dt[which][k] = exp2f(Gs[hi][k] - Gs[lo][k]);
  }
  __syncthreads();

  {
    const int bi = tid >> 4, bj = tid & 15;
    float Ao[6], Po[6], Ai[4], Pi[4];
#pragma unroll
    for (int x = 0; x < 6; ++x) { Ao[x] = 0.f; Po[x] = 0.f; }
#pragma unroll
    for (int x = 0; x < 4; ++x) { Ai[x] = 0.f; Pi[x] = 0.f; }
    auto dot = [](const float4& a, const float4& b) { return a.x * b.x + a.y * b.y + a.z * b.z + a.w * b.w; };
    auto mul = [](const float4& a, const float4& b) { return make_float4(a.x * b.x, a.y * b.y, a.z * b.z, a.w * b.w); };
    auto ex2 = [](const float4& a, const float4& b) {      // 2^min(a - b, 0)
      return make_float4(exp2f(fminf(a.x - b.x, 0.f)), exp2f(fminf(a.y - b.y, 0.f)), exp2f(fminf(a.z - b.z, 0.f)),
                         exp2f(fminf(a.w - b.w, 0.f)));
    };
#pragma unroll 1
    for (int k = 0; k < DD; k += 4) {
      float4 ki[4], qi[4], gi[4];
#pragma unroll
      for (int a = 0; a < 4; ++a) {
        ki[a] = *reinterpret_cast<const float4*>(&Ks[bi + 16 * a][k]);
        qi[a] = *reinterpret_cast<const float4*>(&Qs[bi + 16 * a][k]);
        gi[a] = *reinterpret_cast<const float4*>(&Gs[bi + 16 * a][k]);
      }
      // pairs inside a group; the same column loads give the folded keys km[b] = k_j 2^(R_b' - G_j) of groups 0..2
      float4 km[3], kp[4], qp[4], rr[4];
#pragma unroll
      for (int a = 1; a < 4; ++a) rr[a] = *reinterpret_cast<const float4*>(&Gs[16 * a - 1][k]);      // R_a = R_(a-1)'
#pragma unroll
      for (int a = 0; a < 4; ++a) {
        const float4 kj = *reinterpret_cast<const float4*>(&Ks[bj + 16 * a][k]);
        const float4 gj = *reinterpret_cast<const float4*>(&Gs[bj + 16 * a][k]);
        const float4 t = mul(kj, ex2(gi[a], gj));
        Ai[a] += dot(ki[a], t);
        Pi[a] += dot(qi[a], t);
        if (a < 3) km[a] = mul(kj, ex2(rr[a + 1], gj));
      }
      // pairs across groups: rows of group a >= 1 against columns of groups b < a
#pragma unroll
      for (int a = 1; a < 4; ++a) {
        const float4 e1 = ex2(gi[a], rr[a]);
        kp[a] = mul(ki[a], e1);
        qp[a] = mul(qi[a], e1);
      }
      const float4 d21 = *reinterpret_cast<const float4*>(&Dt[0][k]), d31 = *reinterpret_cast<const float4*>(&Dt[1][k]),
                   d32 = *reinterpret_cast<const float4*>(&Dt[2][k]);
      const float4 t20 = mul(km[0], d21), t30 = mul(km[0], d31), t31 = mul(km[1], d32);
      Ao[0] += dot(kp[1], km[0]); Po[0] += dot(qp[1], km[0]);      // (1, 0)
      Ao[1] += dot(kp[2], t20);   Po[1] += dot(qp[2], t20);        // (2, 0)
      Ao[2] += dot(kp[2], km[1]); Po[2] += dot(qp[2], km[1]);      // (2, 1)
      Ao[3] += dot(kp[3], t30);   Po[3] += dot(qp[3], t30);        // (3, 0)
      Ao[4] += dot(kp[3], t31);   Po[4] += dot(qp[3], t31);        // (3, 1)
      Ao[5] += dot(kp[3], km[2]); Po[5] += dot(qp[3], km[2]);      // (3, 2)
    }
    __syncthreads();      // every pairwise sum is in registers: raw q, k and the running sums are read once more below
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int p = tid + 256 * i, tok = p >> 4, c0 = (p & 15) * 8;
      const float be = bs[tok];
      const float2 v01 = unpack_bf16x2(vreg[i].x), v23 = unpack_bf16x2(vreg[i].y), v45 = unpack_bf16x2(vreg[i].z),
                   v67 = unpack_bf16x2(vreg[i].w);
      const float vv[8] = {v01.x, v01.y, v23.x, v23.y, v45.x, v45.y, v67.x, v67.y};
      float qo[8], ko[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const float q = Qs[tok][c0 + e], k = Ks[tok][c0 + e], gt = Gs[tok][c0 + e];
        const float eg = exp2f(gt), ed = exp2f(Gs[CH - 1][c0 + e] - gt);
        qo[e] = tf32r(eg * q);
        ko[e] = tf32r(ed * k);
        Ks[tok][c0 + e] = tf32r(be * eg * k);
        Qs[tok][c0 + e] = tf32r(be * vv[e]);
      }
      if (tok < nvalid) {
        float* qd = Qg + ((size_t)(r0 + tok) * hv + h) * DD + c0;
        float* kd = Kg + ((size_t)(r0 + tok) * hv + h) * DD + c0;
        *reinterpret_cast<float4*>(qd) = make_float4(qo[0], qo[1], qo[2], qo[3]);
        *reinterpret_cast<float4*>(qd + 4) = make_float4(qo[4], qo[5], qo[6], qo[7]);
        *reinterpret_cast<float4*>(kd) = make_float4(ko[0], ko[1], ko[2], ko[3]);
        *reinterpret_cast<float4*>(kd + 4) = make_float4(ko[4], ko[5], ko[6], ko[7]);
      }
    }
    if (tid < DD) Dg[((size_t)r0 * hv + h) * DD + tid] = exp2f(Gs[CH - 1][tid]);
    __syncthreads();      // the running sums are used up: L takes their place
    // scatter: L strictly below the diagonal (times beta_i), M on and below it, zeros above
#pragma unroll
    for (int a = 0; a < 4; ++a) {
      const int i = bi + 16 * a;
      const float be = bs[i];
#pragma unroll
      for (int b = 0; b < 4; ++b) {
        const int j = bj + 16 * b;
        float lv = 0.f, mv = 0.f;
        if (b == a) {
          lv = bj < bi ? Ai[a] : 0.f;
          mv = bj <= bi ? Pi[a] : 0.f;
        } else if (b < a) {
          const int x = a == 1 ? 0 : (a == 2 ? 1 + b : 3 + b);
          lv = Ao[x];
          mv = Po[x];
        }
        Ls[i][j] = be * lv;
        if (i < nvalid) Mg[((size_t)(r0 + i) * hv + h) * CH + j] = tf32r(mv);
      }
    }
  }
  __syncthreads();      // L complete
  solve_and_project(Ls, Ks, Qs, Wg, Ug, r0, nvalid, hv, h);
}

// grid [HV * 2, seqs], block 256, dynamic shared memory RULE_SMEM bytes. A CTA owns 64 value rows of one head.
// Warps 0..3 keep the state (16 value rows x 128 keys each, as accumulator fragments) and compute U and S1; warps
// 4..7 compute the outputs. Two block barriers per chunk; every operand buffer is refilled right after its product.
constexpr int RULE_SMEM = (CH * LDK * 3 + CH * LDN + CH * LDL + 2 * CH * LDU) * 4;

// KDA: the state's decay over a chunk is a vector over the keys, Gg [.., HV, 128] read at the chunk's first token.
template <bool KDA>
__device__ __forceinline__ void chunk_rule_body(const float* Wg, const float* Qg, const float* Kg, const float* Ug,
                                                const float* Mg, const float* Gg, float* o_raw, uint8_t* state,
                                                const int* lines, const int* cu_q, int seqs, int hv, long long line_bytes,
                                                long long s_offset) {
  pdl_wait();
  extern __shared__ __align__(16) float sm[];
  float (*Ss)[LDK] = reinterpret_cast<float (*)[LDK]>(sm);                                  // state rows (tf32), B[k][n] = Ss[n][k]
  float (*Wc)[LDK] = reinterpret_cast<float (*)[LDK]>(sm + CH * LDK);
  float (*Qc)[LDK] = reinterpret_cast<float (*)[LDK]>(sm + 2 * CH * LDK);
  float (*Kc)[LDN] = reinterpret_cast<float (*)[LDN]>(sm + 3 * CH * LDK);
  float (*Mc)[LDL] = reinterpret_cast<float (*)[LDL]>(sm + 3 * CH * LDK + CH * LDN);
  float (*Uc)[LDU] = reinterpret_cast<float (*)[LDU]>(sm + 3 * CH * LDK + CH * LDN + CH * LDL);              // Ut
  float (*Us)[LDU] = reinterpret_cast<float (*)[LDU]>(sm + 3 * CH * LDK + CH * LDN + CH * LDL + CH * LDU);   // U
  const int s = blockIdx.y;
  if (s >= seqs) return;
  const int h = blockIdx.x >> 1, dv0 = (blockIdx.x & 1) * 64;
  const int q0 = cu_q[s], q1 = cu_q[s + 1];
  if (q1 <= q0) return;
  const int nch = (q1 - q0 + CH - 1) / CH;
  const int line = lines[s];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t4 = lane & 3;

  auto load_wqu = [&](int c) {      // W, Qg (64 x 128) and the CTA's 64 columns of Ut
    const int r0 = q0 + c * CH, nv = min(CH, q1 - r0);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int p = tid + 256 * i, row = p >> 5, c4 = (p & 31) * 4;
      const size_t at = ((size_t)(r0 + min(row, nv - 1)) * hv + h) * DD + c4;
      cp_async16(&Wc[row][c4], Wg + at, row < nv);
      cp_async16(&Qc[row][c4], Qg + at, row < nv);
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int p = tid + 256 * i, row = p >> 4, c4 = (p & 15) * 4;
      cp_async16(&Uc[row][c4], Ug + ((size_t)(r0 + min(row, nv - 1)) * hv + h) * DD + dv0 + c4, row < nv);
    }
  };
  auto load_km = [&](int c) {       // Kd (64 x 128) and M (64 x 64)
    const int r0 = q0 + c * CH, nv = min(CH, q1 - r0);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int p = tid + 256 * i, row = p >> 5, c4 = (p & 31) * 4;
      cp_async16(&Kc[row][c4], Kg + ((size_t)(r0 + min(row, nv - 1)) * hv + h) * DD + c4, row < nv);
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int p = tid + 256 * i, row = p >> 4, c4 = (p & 15) * 4;
      cp_async16(&Mc[row][c4], Mg + ((size_t)(r0 + min(row, nv - 1)) * hv + h) * CH + c4, row < nv);
    }
  };
  load_wqu(0);
  cp_async_commit();
  load_km(0);
  cp_async_commit();

  // the state: warp w < 4 holds value rows dv0 + 16 w + {g, g + 8}, keys 8 nt + {2 t4, 2 t4 + 1}
  float S[16][4];
  float* Sgl = reinterpret_cast<float*>(state + (size_t)line * line_bytes + s_offset) + ((size_t)h * DD + dv0) * DD;
  if (warp < 4) {
#pragma unroll
    for (int nt = 0; nt < 16; ++nt)
#pragma unroll
      for (int hh = 0; hh < 2; ++hh) {
        const int r = 16 * warp + g + 8 * hh, col = 8 * nt + 2 * t4;
        const float2 v = line > 0 ? *reinterpret_cast<const float2*>(Sgl + (size_t)r * DD + col) : make_float2(0.f, 0.f);
        S[nt][2 * hh] = v.x;
        S[nt][2 * hh + 1] = v.y;
        *reinterpret_cast<float2*>(&Ss[r][col]) = make_float2(tf32r(v.x), tf32r(v.y));
      }
  }
  cp_async_wait_all();
  __syncthreads();

  for (int c = 0; c < nch; ++c) {
    const int r0 = q0 + c * CH, nv = min(CH, q1 - r0);
    const float gC = KDA ? 1.f : Gg[(size_t)r0 * hv + h];
    const int wl = warp & 3;
    float2 dk[16];
    if constexpr (KDA) {
      if (warp < 4) {
#pragma unroll
        for (int nt = 0; nt < 16; ++nt)
          dk[nt] = *reinterpret_cast<const float2*>(Gg + ((size_t)r0 * hv + h) * DD + 8 * nt + 2 * t4);
      }
    }
    float acc[8][4];
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
    auto s_at = [&](int k, int n) { return __float_as_uint(Ss[n][k]); };
    if (warp < 4) {
      // U = Ut - W S0^T
      warp_mma<8>(acc, DD / 8, [&](int m, int k) { return __float_as_uint(Wc[16 * wl + m][k]); }, s_at);
#pragma unroll
      for (int nt = 0; nt < 8; ++nt)
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
          const int r = 16 * wl + g + 8 * hh, col = 8 * nt + 2 * t4;
          const float2 ut = *reinterpret_cast<const float2*>(&Uc[r][col]);
          *reinterpret_cast<float2*>(&Us[r][col]) =
              make_float2(tf32r(ut.x - acc[nt][2 * hh]), tf32r(ut.y - acc[nt][2 * hh + 1]));
        }
    } else {
      // Qg S0^T, the first half of the outputs
      warp_mma<8>(acc, DD / 8, [&](int m, int k) { return __float_as_uint(Qc[16 * wl + m][k]); }, s_at);
    }
    cp_async_wait_all();      // Kd and M of this chunk
    __syncthreads();          // U is visible; W, Qg, Ut are free
    if (c + 1 < nch) load_wqu(c + 1);
    cp_async_commit();
    if (warp < 4) {
      // S1 = gC S0 + U^T Kd
#pragma unroll
      for (int nt = 0; nt < 16; ++nt)
#pragma unroll
        for (int j = 0; j < 4; ++j) S[nt][j] *= KDA ? ((j & 1) ? dk[nt].y : dk[nt].x) : gC;
      warp_mma<16>(S, CH / 8, [&](int m, int k) { return __float_as_uint(Us[k][16 * wl + m]); },
                   [&](int k, int n) { return __float_as_uint(Kc[k][n]); });
#pragma unroll
      for (int nt = 0; nt < 16; ++nt)
#pragma unroll
        for (int hh = 0; hh < 2; ++hh)
          *reinterpret_cast<float2*>(&Ss[16 * wl + g + 8 * hh][8 * nt + 2 * t4]) =
              make_float2(tf32r(S[nt][2 * hh]), tf32r(S[nt][2 * hh + 1]));
    } else {
      // O = Qg S0^T + M U; M is lower triangular, the product stops at the diagonal block
      warp_mma<8>(acc, 2 * (wl + 1), [&](int m, int k) { return __float_as_uint(Mc[16 * wl + m][k]); },
                  [&](int k, int n) { return __float_as_uint(Us[k][n]); });
#pragma unroll
      for (int nt = 0; nt < 8; ++nt)
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
          const int r = 16 * wl + g + 8 * hh;
          if (r < nv)
            *reinterpret_cast<float2*>(o_raw + ((size_t)(r0 + r) * hv + h) * DD + dv0 + 8 * nt + 2 * t4) =
                make_float2(acc[nt][2 * hh], acc[nt][2 * hh + 1]);
        }
    }
    cp_async_wait_all();      // W, Qg, Ut of the next chunk
    __syncthreads();          // the new state is in place; Kd, M, U are free
    if (c + 1 < nch) load_km(c + 1);
    cp_async_commit();
  }
  if (warp < 4 && line > 0) {
#pragma unroll
    for (int nt = 0; nt < 16; ++nt)
#pragma unroll
      for (int hh = 0; hh < 2; ++hh)
        *reinterpret_cast<float2*>(Sgl + (size_t)(16 * warp + g + 8 * hh) * DD + 8 * nt + 2 * t4) =
            make_float2(S[nt][2 * hh], S[nt][2 * hh + 1]);
  }
}

extern "C" __global__ void __launch_bounds__(256, 1)
    kern_gdn_chunk_rule_k128_v128(const float* Wg, const float* Qg, const float* Kg, const float* Ug, const float* Mg,
                                  const float* Gg, float* o_raw, uint8_t* state, const int* lines, const int* cu_q, int seqs,
                                  int hv, long long line_bytes, long long s_offset) {
  chunk_rule_body<false>(Wg, Qg, Kg, Ug, Mg, Gg, o_raw, state, lines, cu_q, seqs, hv, line_bytes, s_offset);
}

// The per-key-decay rule (Kimi Delta Attention): same walk, `Dg` [tokens, HV, 128] holds at a chunk's first token the
// decay of every key over the chunk.
extern "C" __global__ void __launch_bounds__(256, 1)
    kern_kda_chunk_rule_k128_v128(const float* Wg, const float* Qg, const float* Kg, const float* Ug, const float* Mg,
                                  const float* Dg, float* o_raw, uint8_t* state, const int* lines, const int* cu_q, int seqs,
                                  int hv, long long line_bytes, long long s_offset) {
  chunk_rule_body<true>(Wg, Qg, Kg, Ug, Mg, Dg, o_raw, state, lines, cu_q, seqs, hv, line_bytes, s_offset);
}
