// Element codecs for comparisons: bytes of any manifest dtype <-> double, and the ULP distance
// between two encodings (0 for bit-identical, +0 vs -0 counts 0, NaN against anything counts max).
// Reference: crates/kern-manifest/src/values.rs:9-135.
#pragma once
#include <cmath>
#include <cstring>
#include <string>
#include <vector>

#include "types.hpp"

namespace kern {
namespace values {

inline float bf16_to_f32(uint16_t h) { uint32_t u = (uint32_t)h << 16; float f; std::memcpy(&f, &u, 4); return f; }
inline uint16_t f32_to_bf16(float f) {
  uint32_t u; std::memcpy(&u, &f, 4);
  if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x40);   // quiet NaN
  u += 0x7fffu + ((u >> 16) & 1);                                             // round to nearest even
  return (uint16_t)(u >> 16);
}
inline float f16_to_f32(uint16_t h) {
  const uint32_t s = (h >> 15) & 1, e = (h >> 10) & 31, m = h & 1023;
  float v;
  if (e == 0) v = std::ldexp((float)m, -24);
  else if (e == 31) v = m ? NAN : INFINITY;
  else v = std::ldexp((float)(m | 1024), (int)e - 25);
  return s ? -v : v;
}
inline uint16_t f32_to_f16(float f) {
  if (std::isnan(f)) return 0x7e00;
  const uint16_t s = std::signbit(f) ? 0x8000 : 0;
  float a = std::fabs(f);
  if (a >= 65520.f) return s | 0x7c00;
  if (a < std::ldexp(1.f, -25)) return s;
  int e;
  float fr = std::frexp(a, &e);   // a = fr * 2^e, fr in [0.5, 1)
  int exp = e + 14;               // biased exponent for 1.xxx form
  if (exp <= 0) {                 // subnormal
    uint32_t m = (uint32_t)std::nearbyint(std::ldexp(a, 24));
    return s | (uint16_t)m;
  }
  uint32_t m = (uint32_t)std::nearbyint(std::ldexp(fr, 11)) - 1024;   // 10-bit mantissa, may carry to 1024
  uint32_t bits = ((uint32_t)exp << 10) + m;
  return s | (uint16_t)bits;
}
// OCP fp8 e4m3 (finite-only, 0x7f / 0xff NaN, max 448)
inline float e4m3_to_f32(uint8_t b) {
  const uint32_t s = b >> 7, e = (b >> 3) & 15, m = b & 7;
  float v;
  if (e == 15 && m == 7) v = NAN;
  else if (e == 0) v = std::ldexp((float)m, -9);
  else v = std::ldexp((float)(m | 8), (int)e - 10);
  return s ? -v : v;
}
inline uint8_t f32_to_e4m3(float f) {
  if (std::isnan(f)) return 0x7f;
  const uint8_t s = std::signbit(f) ? 0x80 : 0;
  float a = std::fmin(std::fabs(f), 448.f);
  uint8_t best = 0;
  float bd = INFINITY;
  for (int c = 0; c < 0x7f; ++c) {   // 127 finite magnitudes: exact nearest, ties to even code
    float d = std::fabs(e4m3_to_f32((uint8_t)c) - a);
    if (d < bd || (d == bd && !(c & 1))) { bd = d; best = (uint8_t)c; }
  }
  return s | best;
}
// e8m0: an unsigned power-of-two scale, 2^(b - 127); 0xff is NaN
inline float e8m0_to_f32(uint8_t b) { return b == 0xff ? NAN : std::ldexp(1.f, (int)b - 127); }
inline uint8_t f32_to_e8m0(float f) {
  if (std::isnan(f) || f <= 0) return f == 0 ? 0 : 0xff;
  int e = (int)std::nearbyint(std::log2(f)) + 127;
  return (uint8_t)std::min(254, std::max(0, e));
}
// fp4 e2m1 (the MXFP4 element): magnitudes 0, .5, 1, 1.5, 2, 3, 4, 6
inline float e2m1_to_f32(uint8_t nib) {
  static const float t[8] = {0.f, 0.5f, 1.f, 1.5f, 2.f, 3.f, 4.f, 6.f};
  float v = t[nib & 7];
  return (nib & 8) ? -v : v;
}

inline std::vector<double> decode(DType dt, const std::string& bytes) {
  const size_t n = bytes.size() / dtype_bytes(dt);
  std::vector<double> out(n);
  const uint8_t* p = reinterpret_cast<const uint8_t*>(bytes.data());
  for (size_t i = 0; i < n; ++i) {
    switch (dt) {
      case DType::bf16: { uint16_t h; std::memcpy(&h, p + 2 * i, 2); out[i] = bf16_to_f32(h); break; }
      case DType::f16: { uint16_t h; std::memcpy(&h, p + 2 * i, 2); out[i] = f16_to_f32(h); break; }
      case DType::f32: { float f; std::memcpy(&f, p + 4 * i, 4); out[i] = f; break; }
      case DType::fp8e4m3: out[i] = e4m3_to_f32(p[i]); break;
      case DType::fp8e8m0: out[i] = e8m0_to_f32(p[i]); break;
      case DType::i8: out[i] = (int8_t)p[i]; break;
      case DType::u8: out[i] = p[i]; break;
      case DType::i32: { int32_t v; std::memcpy(&v, p + 4 * i, 4); out[i] = v; break; }
      case DType::u32: { uint32_t v; std::memcpy(&v, p + 4 * i, 4); out[i] = v; break; }
      case DType::i64: { int64_t v; std::memcpy(&v, p + 8 * i, 8); out[i] = (double)v; break; }
      case DType::u64: { uint64_t v; std::memcpy(&v, p + 8 * i, 8); out[i] = (double)v; break; }
    }
  }
  return out;
}
inline std::string encode(DType dt, const std::vector<double>& v) {
  std::string out(v.size() * dtype_bytes(dt), '\0');
  uint8_t* p = reinterpret_cast<uint8_t*>(&out[0]);
  for (size_t i = 0; i < v.size(); ++i) {
    switch (dt) {
      case DType::bf16: { uint16_t h = f32_to_bf16((float)v[i]); std::memcpy(p + 2 * i, &h, 2); break; }
      case DType::f16: { uint16_t h = f32_to_f16((float)v[i]); std::memcpy(p + 2 * i, &h, 2); break; }
      case DType::f32: { float f = (float)v[i]; std::memcpy(p + 4 * i, &f, 4); break; }
      case DType::fp8e4m3: p[i] = f32_to_e4m3((float)v[i]); break;
      case DType::fp8e8m0: p[i] = f32_to_e8m0((float)v[i]); break;
      case DType::i8: p[i] = (uint8_t)(int8_t)v[i]; break;
      case DType::u8: p[i] = (uint8_t)v[i]; break;
      case DType::i32: { int32_t x = (int32_t)v[i]; std::memcpy(p + 4 * i, &x, 4); break; }
      case DType::u32: { uint32_t x = (uint32_t)v[i]; std::memcpy(p + 4 * i, &x, 4); break; }
      case DType::i64: { int64_t x = (int64_t)v[i]; std::memcpy(p + 8 * i, &x, 8); break; }
      case DType::u64: { uint64_t x = (uint64_t)v[i]; std::memcpy(p + 8 * i, &x, 8); break; }
    }
  }
  return out;
}

// order-preserving integer key of a sign-magnitude float encoding of `bits` bits
inline int64_t ordered_key(uint64_t raw, int bits) {
  const uint64_t sign = 1ull << (bits - 1);
  return (raw & sign) ? -(int64_t)(raw & (sign - 1)) : (int64_t)raw;
}
inline uint64_t ulp_distance_one(DType dt, const uint8_t* a, const uint8_t* b) {
  auto raw = [&](const uint8_t* p) { uint64_t r = 0; std::memcpy(&r, p, dtype_bytes(dt)); return r; };
  const uint64_t ra = raw(a), rb = raw(b);
  if (ra == rb) return 0;
  if (dtype_is_int(dt)) {
    std::string sa(reinterpret_cast<const char*>(a), dtype_bytes(dt)), sb(reinterpret_cast<const char*>(b), dtype_bytes(dt));
    double da = decode(dt, sa)[0], db = decode(dt, sb)[0];
    return (uint64_t)std::fabs(da - db);
  }
  std::string sa(reinterpret_cast<const char*>(a), dtype_bytes(dt)), sb(reinterpret_cast<const char*>(b), dtype_bytes(dt));
  const double da = decode(dt, sa)[0], db = decode(dt, sb)[0];
  if (std::isnan(da) || std::isnan(db)) return (std::isnan(da) && std::isnan(db)) ? 0 : UINT64_MAX;
  if (dt == DType::fp8e8m0) return ra > rb ? ra - rb : rb - ra;
  const int bits = (int)dtype_bytes(dt) * 8;
  const int64_t ka = ordered_key(ra, bits), kb = ordered_key(rb, bits);
  return (uint64_t)(ka > kb ? ka - kb : kb - ka);
}
inline uint64_t max_ulp_distance(DType dt, const std::string& a, const std::string& b) {
  const size_t w = dtype_bytes(dt), n = std::min(a.size(), b.size()) / w;
  uint64_t worst = a.size() == b.size() ? 0 : UINT64_MAX;
  for (size_t i = 0; i < n; ++i)
    worst = std::max(worst, ulp_distance_one(dt, reinterpret_cast<const uint8_t*>(a.data()) + i * w,
                                             reinterpret_cast<const uint8_t*>(b.data()) + i * w));
  return worst;
}

}  // namespace values
}  // namespace kern
