// Host-side converters for block-scaled checkpoint formats, exported with C linkage for ctypes. They run once per tensor
// when a quantised checkpoint is loaded or written, over tens of GB, which is why the reference has compiled (Triton)
// converters for them (paddleformers/utils/upcast_downcast_triton.py:56-355, paddleformers/quantization/checkpoint_dequant.py:
// 277-355).
//
//   pfb_mxfp4_dequant_bf16     groups of 32 e2m1 values (two per byte, low nibble first) x 2^(E8M0 - 127) -> bf16
//   pfb_mxfp4_quant            fp32 -> e2m1 groups + E8M0 exponents (round to nearest, ties towards zero)
//   pfb_mxfp8_dequant_bf16     groups of 32 e4m3 bytes x 2^(E8M0 - 127) -> bf16
//   pfb_mxfp8_quant            fp32 -> e4m3 groups + E8M0 exponents
//   pfb_fp8_block_dequant_bf16 e4m3 [N, K] x one fp32 scale per block x block tile -> bf16
//
// Work is split over std::threads by groups / rows; every function is a pure map, so the result does not depend on the
// number of threads.
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <thread>
#include <vector>

namespace {

const float kE2M1[16] = {0.0f, 0.5f, 1.0f, 1.5f, 2.0f, 3.0f, 4.0f, 6.0f, -0.0f, -0.5f, -1.0f, -1.5f, -2.0f, -3.0f, -4.0f, -6.0f};

inline uint16_t float_to_bf16(float f) {
  uint32_t u;
  std::memcpy(&u, &f, 4);
  if ((u & 0x7fffffffu) > 0x7f800000u) return static_cast<uint16_t>((u >> 16) | 0x40);  // NaN stays NaN
  u += 0x7fffu + ((u >> 16) & 1u);                                                        // round to nearest even
  return static_cast<uint16_t>(u >> 16);
}

inline float e8m0_to_float(uint8_t e) {
  // 2^(e - 127); e = 255 is NaN in the format, e = 0 is 2^-127 (a float subnormal)
  if (e == 255) return std::nanf("");
  return std::ldexp(1.0f, static_cast<int>(e) - 127);
}

inline float e4m3_to_float(uint8_t b) {
  const int sign = b >> 7, exp = (b >> 3) & 0xF, man = b & 7;
  float v;
  if (exp == 0) v = std::ldexp(static_cast<float>(man), -9);                  // subnormal: man * 2^-3 * 2^-6
  else if (exp == 15 && man == 7) v = std::nanf("");                          // e4m3fn: only S.1111.111 is NaN
  else v = std::ldexp(1.0f + man / 8.0f, exp - 7);
  return sign ? -v : v;
}

inline uint8_t float_to_e4m3(float f) {
  // round to nearest even, saturating at +-448
  if (std::isnan(f)) return 0x7f;
  const uint8_t sign = std::signbit(f) ? 0x80 : 0;
  float a = std::fabs(f);
  if (a >= 448.0f) return sign | 0x7e;
  if (a < std::ldexp(1.0f, -10)) return sign;                                 // below half of the smallest subnormal
  int e;
  std::frexp(a, &e);                                                          // a = m * 2^e, m in [0.5, 1)
  int exp = e - 1;                                                            // a = 1.xxx * 2^exp
  if (exp < -6) exp = -6;                                                     // subnormal range shares the exponent -6
  const float step = std::ldexp(1.0f, exp - 3);                               // spacing of representable values
  float q = std::nearbyint(a / step);                                         // default rounding mode: to nearest even
  float v = q * step;
  if (v >= 448.0f) return sign | 0x7e;
  int e2;
  std::frexp(v, &e2);
  int vexp = e2 - 1;
  if (v < std::ldexp(1.0f, -6)) return sign | static_cast<uint8_t>(std::lround(std::ldexp(v, 9)));
  const int man = static_cast<int>(std::lround((std::ldexp(v, -vexp) - 1.0f) * 8.0f));
  return sign | static_cast<uint8_t>(((vexp + 7) << 3) | man);
}

// exponent k such that amax / limit <= 2^k, exactly (no log2 rounding)
inline int ceil_log2_ratio(float amax, float limit) {
  int k;
  const float m = std::frexp(amax / limit, &k);                               // amax/limit = m * 2^k, m in [0.5, 1)
  return m > 0.5f ? k : k - 1;
}

template <class Fn>
void parallel_for(int64_t n, int64_t grain, Fn fn) {
  unsigned hw = std::thread::hardware_concurrency();
  int64_t workers = std::min<int64_t>(hw ? std::min(hw, 16u) : 4, std::max<int64_t>(n / std::max<int64_t>(grain, 1), 1));
  if (workers <= 1) { fn(0, n); return; }
  std::vector<std::thread> pool;
  const int64_t per = (n + workers - 1) / workers;
  for (int64_t w = 0; w < workers; ++w) {
    const int64_t lo = w * per, hi = std::min(n, lo + per);
    if (lo >= hi) break;
    pool.emplace_back([=] { fn(lo, hi); });
  }
  for (auto& t : pool) t.join();
}

}  // namespace

extern "C" {

void pfb_mxfp4_dequant_bf16(const uint8_t* blocks, const uint8_t* scales, uint16_t* out, int64_t n_groups) {
  parallel_for(n_groups, 4096, [=](int64_t lo, int64_t hi) {
    for (int64_t g = lo; g < hi; ++g) {
      const float s = e8m0_to_float(scales[g]);
      const uint8_t* b = blocks + g * 16;
      uint16_t* o = out + g * 32;
      for (int i = 0; i < 16; ++i) {
        o[2 * i] = float_to_bf16(kE2M1[b[i] & 0xF] * s);
        o[2 * i + 1] = float_to_bf16(kE2M1[b[i] >> 4] * s);
      }
    }
  });
}

void pfb_mxfp4_quant(const float* x, uint8_t* blocks, uint8_t* scales, int64_t n_groups) {
  parallel_for(n_groups, 4096, [=](int64_t lo, int64_t hi) {
    for (int64_t g = lo; g < hi; ++g) {
      const float* v = x + g * 32;
      float amax = 0.0f;
      for (int i = 0; i < 32; ++i) amax = std::max(amax, std::fabs(v[i]));
      amax = std::max(amax, std::ldexp(1.0f, -126));
      int e = ceil_log2_ratio(amax, 6.0f);
      e = std::min(std::max(e, -127), 127);
      scales[g] = static_cast<uint8_t>(e + 127);
      const float inv = std::ldexp(1.0f, -e);
      uint8_t* b = blocks + g * 16;
      for (int i = 0; i < 32; ++i) {
        const float s = v[i] * inv, a = std::fabs(s);
        int best = 0;
        float bd = a;                                       // distance to 0
        for (int k = 1; k < 8; ++k) {
          const float d = std::fabs(a - kE2M1[k]);
          if (d < bd) { bd = d; best = k; }                 // strict: ties keep the smaller magnitude
        }
        const uint8_t code = static_cast<uint8_t>(best == 0 ? 0 : (best | (s < 0 ? 8 : 0)));
        if (i & 1) b[i >> 1] |= static_cast<uint8_t>(code << 4); else b[i >> 1] = code;
      }
    }
  });
}

void pfb_mxfp8_dequant_bf16(const uint8_t* q, const uint8_t* scales, uint16_t* out, int64_t n_groups) {
  parallel_for(n_groups, 4096, [=](int64_t lo, int64_t hi) {
    for (int64_t g = lo; g < hi; ++g) {
      const float s = e8m0_to_float(scales[g]);
      for (int i = 0; i < 32; ++i) out[g * 32 + i] = float_to_bf16(e4m3_to_float(q[g * 32 + i]) * s);
    }
  });
}

void pfb_mxfp8_quant(const float* x, uint8_t* q, uint8_t* scales, int64_t n_groups) {
  parallel_for(n_groups, 4096, [=](int64_t lo, int64_t hi) {
    for (int64_t g = lo; g < hi; ++g) {
      const float* v = x + g * 32;
      float amax = 0.0f;
      for (int i = 0; i < 32; ++i) amax = std::max(amax, std::fabs(v[i]));
      amax = std::max(amax, std::ldexp(1.0f, -126));
      int e = ceil_log2_ratio(amax, 448.0f);
      e = std::min(std::max(e, -127), 127);
      scales[g] = static_cast<uint8_t>(e + 127);
      const float inv = std::ldexp(1.0f, -e);
      for (int i = 0; i < 32; ++i) q[g * 32 + i] = float_to_e4m3(v[i] * inv);
    }
  });
}

// w: e4m3 bytes [N, K] row-major; scale: fp32 [ceil(N / block), ceil(K / block)]
void pfb_fp8_block_dequant_bf16(const uint8_t* w, const float* scale, uint16_t* out, int64_t N, int64_t K, int64_t block) {
  const int64_t kb = (K + block - 1) / block;
  parallel_for(N, 64, [=](int64_t lo, int64_t hi) {
    for (int64_t r = lo; r < hi; ++r) {
      const float* srow = scale + (r / block) * kb;
      for (int64_t c = 0; c < K; ++c) out[r * K + c] = float_to_bf16(e4m3_to_float(w[r * K + c]) * srow[c / block]);
    }
  });
}

}  // extern "C"
