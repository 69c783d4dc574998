// Seeded random weights as a pure function of (key, element index): the same bits on the GPU and
// in the NumPy statement of the same arithmetic (llmario_b200/weights/random_normal.py).
//
// The reference's own fixture generator is a pure function of the index as well
// (crates/engine/model/src/forward.rs:873-881: an integer hash of the index per tensor).  Here the
// hash feeds a Box-Muller transform whose logarithm, square root, sine and cosine are written out
// in IEEE double operations that round the same everywhere (add, multiply, divide, square root;
// no fused multiply-add, no library function), so a model made on the device can be rebuilt
// value by value on any host.
//
//   h      = mix(key + (i + 1) * 0x9E3779B97F4A7C15)              (the finalizer of splitmix64)
//   u1     = ((h >> 32) + 1) / 2^32            in (0, 1]
//   turn   = (h & 0xffffffff) / 2^32           in [0, 1)
//   z      = sqrt(-2 ln u1) * cos(2 pi turn)
//   value  = float32(mean + std * z), then bfloat16 (nearest even) if the tensor is 16-bit
#include "common.cuh"

namespace {

__host__ __device__ inline unsigned long long mix64(unsigned long long z) {
  z ^= z >> 30;
  z *= 0xBF58476D1CE4E5B9ULL;
  z ^= z >> 27;
  z *= 0x94D049BB133111EBULL;
  z ^= z >> 31;
  return z;
}

__device__ inline double mul(double a, double b) { return __dmul_rn(a, b); }
__device__ inline double add(double a, double b) { return __dadd_rn(a, b); }

// ln(n / 2^32) for an integer 1 <= n <= 2^32: n = m * 2^e with m in (1/sqrt 2, sqrt 2], then
// ln m = 2 atanh(s), s = (m - 1) / (m + 1), as an odd series to s^21 (|s| < 0.1716).  Never positive.
__device__ inline double ln_unit(unsigned long long n) {
  int e = 63 - __clzll((long long)n);
  double m = mul((double)n, __longlong_as_double((long long)(1023 - e) << 52));   // exact: a power of two
  if (m > 1.4142135623730951) {
    m = mul(m, 0.5);
    e += 1;
  }
  const double s = __ddiv_rn(add(m, -1.0), add(m, 1.0));
  const double s2 = mul(s, s);
  double p = 1.0 / 21.0;
  p = add(mul(p, s2), 1.0 / 19.0);
  p = add(mul(p, s2), 1.0 / 17.0);
  p = add(mul(p, s2), 1.0 / 15.0);
  p = add(mul(p, s2), 1.0 / 13.0);
  p = add(mul(p, s2), 1.0 / 11.0);
  p = add(mul(p, s2), 1.0 / 9.0);
  p = add(mul(p, s2), 1.0 / 7.0);
  p = add(mul(p, s2), 1.0 / 5.0);
  p = add(mul(p, s2), 1.0 / 3.0);
  p = add(mul(p, s2), 1.0);
  return add(mul((double)(e - 32), 0.6931471805599453), mul(mul(2.0, s), p));
}

// cos(2 pi k / 2^32): the top two bits of k choose the quarter turn, the rest is x in [0, pi/2),
// where cos and sin are Taylor polynomials to x^22 and x^23.
__device__ inline double cos_turn(unsigned int k) {
  const int quarter = (int)(k >> 30);
  const double x = mul(mul((double)(k & 0x3fffffffu), 9.313225746154785e-10 /* 2^-30 */), 1.5707963267948966);
  const double x2 = mul(x, x);
  double r;
  if ((quarter & 1) == 0) {   // +-cos x
    double p = -1.0 / 1124000727777607680000.0;               // -1/22!
    p = add(mul(p, x2), 1.0 / 2432902008176640000.0);         //  1/20!
    p = add(mul(p, x2), -1.0 / 6402373705728000.0);           // -1/18!
    p = add(mul(p, x2), 1.0 / 20922789888000.0);              //  1/16!
    p = add(mul(p, x2), -1.0 / 87178291200.0);                // -1/14!
    p = add(mul(p, x2), 1.0 / 479001600.0);                   //  1/12!
    p = add(mul(p, x2), -1.0 / 3628800.0);                    // -1/10!
    p = add(mul(p, x2), 1.0 / 40320.0);                       //  1/8!
    p = add(mul(p, x2), -1.0 / 720.0);                        // -1/6!
    p = add(mul(p, x2), 1.0 / 24.0);
    p = add(mul(p, x2), -0.5);
    r = add(mul(p, x2), 1.0);
  } else {                    // +-sin x
    double p = -1.0 / 25852016738884976640000.0;              // -1/23!
    p = add(mul(p, x2), 1.0 / 51090942171709440000.0);        //  1/21!
    p = add(mul(p, x2), -1.0 / 121645100408832000.0);         // -1/19!
    p = add(mul(p, x2), 1.0 / 355687428096000.0);             //  1/17!
    p = add(mul(p, x2), -1.0 / 1307674368000.0);              // -1/15!
    p = add(mul(p, x2), 1.0 / 6227020800.0);                  //  1/13!
    p = add(mul(p, x2), -1.0 / 39916800.0);                   // -1/11!
    p = add(mul(p, x2), 1.0 / 362880.0);                      //  1/9!
    p = add(mul(p, x2), -1.0 / 5040.0);                       // -1/7!
    p = add(mul(p, x2), 1.0 / 120.0);
    p = add(mul(p, x2), -1.0 / 6.0);
    p = add(mul(p, x2), 1.0);
    r = mul(p, x);
  }
  // quarter 0: cos x; 1: cos(x + pi/2) = -sin x; 2: -cos x; 3: sin x
  return (quarter == 1 || quarter == 2) ? -r : r;
}

template <typename T>
__global__ void random_normal_kernel(T* __restrict__ out, long long n, unsigned long long key, double mean,
                                     double std, long long first) {
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    const unsigned long long h = mix64(key + (unsigned long long)(first + i + 1) * 0x9E3779B97F4A7C15ULL);
    const double ln_u = ln_unit((h >> 32) + 1ULL);
    const double radius = __dsqrt_rn(mul(-2.0, ln_u));
    const double z = mul(radius, cos_turn((unsigned int)(h & 0xffffffffULL)));
    out[i] = from_f32<T>(__double2float_rn(add(mean, mul(std, z))));
  }
}

}  // namespace

// out[i] = mean + std * normal(key, first + i) for i < n, as float32 or bfloat16.
LLM_EXPORT int llm_random_normal(void* out, int dtype, long long n, unsigned long long key, double mean,
                                 double std, long long first, cudaStream_t stream) {
  if (n <= 0) return 0;
  const int threads = 256;
  const int blocks = (int)((n + threads - 1) / threads < 148 * 16 ? (n + threads - 1) / threads : 148 * 16);
  if (dtype == LLM_F32)
    random_normal_kernel<float><<<blocks, threads, 0, stream>>>((float*)out, n, key, mean, std, first);
  else if (dtype == LLM_BF16)
    random_normal_kernel<bf16><<<blocks, threads, 0, stream>>>((bf16*)out, n, key, mean, std, first);
  else
    return LLM_ERR_UNSUPPORTED;
  return launch_status();
}
