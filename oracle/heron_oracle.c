/*
 * heron_oracle.c — CPU restatement of the reference's operator math.  TEST INFRASTRUCTURE ONLY.
 *
 * Only the test-suite, the smoke check and the benchmark's cpu-baseline / reference legs may
 * call into this file; the product path (heron_b200/) never does.
 *
 * PARITY UNPINNED: the reference holds no golden tensor values, known-answer tests or fixtures
 * for these operators (it never checks numerical results: Task.set_verify_func at
 * task/task.py:91-96 has no caller), and it cannot run in this environment (it needs Apache TVM,
 * which is neither vendored nor pinned: requirements.txt:1-4, README.md:25,38).  What pins this
 * file is the arithmetic of the reference's te.compute bodies, restated below one by one, plus an
 * independent numpy restatement checked against it by the tests.
 *
 * Scalar loops on purpose: the order of summation is the textbook one, integers accumulate
 * exactly in int32 (two's complement, as the reference's `astype("int32")` products do), and
 * fp16 inputs are widened exactly and accumulated in double.
 */
#include <stdint.h>
#include <stddef.h>
#include <string.h>
#include <math.h>

/* ---- IEEE binary16 <-> float, exact / round-to-nearest-even --------------------------------- */
static float half_to_float(uint16_t h) {
  const uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
  uint32_t exp = (h >> 10) & 0x1Fu;
  uint32_t man = h & 0x3FFu;
  uint32_t bits;
  if (exp == 0) {
    if (man == 0) {
      bits = sign;
    } else { /* subnormal: renormalise */
      int e = -1;
      do { man <<= 1; ++e; } while ((man & 0x400u) == 0);
      man &= 0x3FFu;
      bits = sign | ((uint32_t)(127 - 15 - e) << 23) | (man << 13);
    }
  } else if (exp == 31) {
    bits = sign | 0x7F800000u | (man << 13);
  } else {
    bits = sign | ((exp + (127 - 15)) << 23) | (man << 13);
  }
  float f;
  memcpy(&f, &bits, sizeof f);
  return f;
}

static uint16_t float_to_half_rn(float f) {
  uint32_t x;
  memcpy(&x, &f, sizeof x);
  const uint16_t sign = (uint16_t)((x >> 16) & 0x8000u);
  const uint32_t absx = x & 0x7FFFFFFFu;
  if (absx >= 0x7F800000u) /* inf / nan */
    return (uint16_t)(sign | 0x7C00u | ((absx > 0x7F800000u) ? 0x200u : 0u));
  if (absx >= 0x477FF000u) /* rounds to >= 65520 -> inf */
    return (uint16_t)(sign | 0x7C00u);
  if (absx < 0x33000001u) /* below half of the smallest subnormal */
    return sign;
  int exp = (int)(absx >> 23) - 127;
  uint32_t man = (absx & 0x7FFFFFu) | 0x800000u;
  int shift;
  uint32_t base;
  if (exp < -14) { /* subnormal result */
    shift = 13 + (-14 - exp);
    base = 0;
  } else {
    shift = 13;
    base = (uint32_t)(exp + 15) << 10;
    man &= 0x7FFFFFu;
  }
  uint32_t q = man >> shift;
  const uint32_t rem = man & ((1u << shift) - 1u);
  const uint32_t half = 1u << (shift - 1);
  if (rem > half || (rem == half && (q & 1u))) ++q;
  return (uint16_t)(sign | (base + q)); /* a carry out of the mantissa bumps the exponent */
}

uint16_t oracle_float_to_half(float f) { return float_to_half_rn(f); }
float oracle_half_to_float(uint16_t h) { return half_to_float(h); }

static inline int32_t load_i8(const void* p, size_t i, int is_signed) {
  return is_signed ? (int32_t)((const int8_t*)p)[i] : (int32_t)((const uint8_t*)p)[i];
}

/*
 * GEMM, integer: out[i,j] = sum_k int32(A[i,k]) * int32(B[j,k]).
 * Follows ops/x86/dense.py:14-18 (A uint8, B int8) and ops/cuda/dense.py:12-17 with
 * out_dtype = int32 (cast to the output type before the multiply, line 14).
 */
void oracle_gemm_i8(const void* A, const void* B, int32_t* C, int M, int K, int N, int a_signed,
                    int b_signed) {
  for (int i = 0; i < M; ++i)
    for (int j = 0; j < N; ++j) {
      int32_t acc = 0;
      for (int k = 0; k < K; ++k)
        acc += load_i8(A, (size_t)i * K + k, a_signed) * load_i8(B, (size_t)j * K + k, b_signed);
      C[(size_t)i * N + j] = acc;
    }
}

/* Batched GEMM, integer: ops/x86/batch_matmul.py:15-20, ops/cuda/batch_matmul.py:14-19. */
void oracle_bmm_i8(const void* A, const void* B, int32_t* C, int batch, int M, int K, int N,
                   int a_signed, int b_signed) {
  for (int b = 0; b < batch; ++b)
    oracle_gemm_i8((const uint8_t*)A + (size_t)b * M * K, (const uint8_t*)B + (size_t)b * N * K,
                   C + (size_t)b * M * N, M, K, N, a_signed, b_signed);
}

/*
 * GEMM, fp16 inputs (raw binary16 bit patterns): ops/cuda/dense.py:12-17 with out_dtype float32.
 * Accumulates in double over exactly widened inputs; writes float.
 */
void oracle_gemm_f16(const uint16_t* A, const uint16_t* B, float* C, int M, int K, int N) {
  for (int i = 0; i < M; ++i)
    for (int j = 0; j < N; ++j) {
      double acc = 0.0;
      for (int k = 0; k < K; ++k)
        acc += (double)half_to_float(A[(size_t)i * K + k]) * (double)half_to_float(B[(size_t)j * K + k]);
      C[(size_t)i * N + j] = (float)acc;
    }
}

void oracle_bmm_f16(const uint16_t* A, const uint16_t* B, float* C, int batch, int M, int K, int N) {
  for (int b = 0; b < batch; ++b)
    oracle_gemm_f16(A + (size_t)b * M * K, B + (size_t)b * N * K, C + (size_t)b * M * N, M, K, N);
}

/* Output extent of the padded, dilated, strided window: ops/cuda/conv2d.py:165-175. */
int oracle_conv_out_extent(int in, int k, int stride, int pad, int dil) {
  const int span = (k - 1) * dil + 1;
  return (in - span + 2 * pad) / stride + 1;
}

/*
 * NHWC conv, integer: ops/cuda/conv2d.py:168-196 (HWIO filter) with integer dtypes; the same sum
 * as ops/x86/conv2d_int8.py:74-93 once the packed filter is indexed logically.
 *   out[n,y,x,f] = sum_{ry,rx,rc} pad(in)[n, y*sh+ry*dh, x*sw+rx*dw, rc] * w[ry,rx,rc,f]
 * `pad` zeros on all four sides (an int padding in get_pad_tuple, ops/cuda/conv2d.py:170-172).
 */
void oracle_conv2d_nhwc_i8(const void* in, const void* w, int32_t* out, int N, int H, int W, int CI,
                           int CO, int KH, int KW, int sh, int sw, int pad, int dh, int dw,
                           int in_signed, int w_signed) {
  const int HO = oracle_conv_out_extent(H, KH, sh, pad, dh);
  const int WO = oracle_conv_out_extent(W, KW, sw, pad, dw);
  for (int n = 0; n < N; ++n)
    for (int y = 0; y < HO; ++y)
      for (int x = 0; x < WO; ++x) {
        int32_t* o = out + (((size_t)n * HO + y) * WO + x) * CO;
        for (int f = 0; f < CO; ++f) o[f] = 0;
        for (int ry = 0; ry < KH; ++ry) {
          const int iy = y * sh + ry * dh - pad;
          if (iy < 0 || iy >= H) continue;
          for (int rx = 0; rx < KW; ++rx) {
            const int ix = x * sw + rx * dw - pad;
            if (ix < 0 || ix >= W) continue;
            const size_t ibase = (((size_t)n * H + iy) * W + ix) * CI;
            const size_t wbase = ((size_t)ry * KW + rx) * CI * CO;
            for (int rc = 0; rc < CI; ++rc) {
              const int32_t a = load_i8(in, ibase + rc, in_signed);
              for (int f = 0; f < CO; ++f)
                o[f] += a * load_i8(w, wbase + (size_t)rc * CO + f, w_signed);
            }
          }
        }
      }
}

/*
 * The x86 operator with its own packed filter (ops/x86/conv2d_int8.py:36-50,74-93):
 * w_packed[(oc_chunk, ry, rx, ic_chunk, oc_block, ic_block)], shape (CO/sco,KH,KW,CI/4,sco,4);
 * input uint8, filter int8, output int32 (N,HO,WO,CO/sco,sco).
 */
void oracle_conv2d_nhwc_packed(const uint8_t* in, const int8_t* wp, int32_t* out, int N, int H,
                               int W, int CI, int CO, int KH, int KW, int sh, int sw, int pad,
                               int dh, int dw, int sco) {
  const int HO = oracle_conv_out_extent(H, KH, sh, pad, dh);
  const int WO = oracle_conv_out_extent(W, KW, sw, pad, dw);
  const int sci = 4;
  for (int n = 0; n < N; ++n)
    for (int y = 0; y < HO; ++y)
      for (int x = 0; x < WO; ++x)
        for (int occ = 0; occ < CO / sco; ++occ)
          for (int ocb = 0; ocb < sco; ++ocb) {
            int32_t acc = 0;
            for (int ry = 0; ry < KH; ++ry) {
              const int iy = y * sh + ry * dh - pad;
              if (iy < 0 || iy >= H) continue;
              for (int rx = 0; rx < KW; ++rx) {
                const int ix = x * sw + rx * dw - pad;
                if (ix < 0 || ix >= W) continue;
                for (int icc = 0; icc < CI / sci; ++icc)
                  for (int icb = 0; icb < sci; ++icb) {
                    const int32_t a = in[(((size_t)n * H + iy) * W + ix) * CI + icc * sci + icb];
                    const int32_t b =
                        wp[(((((size_t)occ * KH + ry) * KW + rx) * (CI / sci) + icc) * sco + ocb) * sci + icb];
                    acc += a * b;
                  }
              }
            }
            out[((((size_t)n * HO + y) * WO + x) * (CO / sco) + occ) * sco + ocb] = acc;
          }
}

/*
 * NHWC conv, fp16 inputs (binary16 bit patterns), double accumulation.  out_half = 0 writes
 * float to `out`; out_half = 1 rounds the double sum to float then to binary16 (RN-even) and
 * writes uint16_t — "fp32 accumulate, fp16 output" of ops/cuda/conv2d.py:182-196.
 */
void oracle_conv2d_nhwc_f16(const uint16_t* in, const uint16_t* w, void* out, int N, int H, int W,
                            int CI, int CO, int KH, int KW, int sh, int sw, int pad, int dh, int dw,
                            int out_half) {
  const int HO = oracle_conv_out_extent(H, KH, sh, pad, dh);
  const int WO = oracle_conv_out_extent(W, KW, sw, pad, dw);
  double acc[4096];
  if (CO > 4096) return;
  for (int n = 0; n < N; ++n)
    for (int y = 0; y < HO; ++y)
      for (int x = 0; x < WO; ++x) {
        for (int f = 0; f < CO; ++f) acc[f] = 0.0;
        for (int ry = 0; ry < KH; ++ry) {
          const int iy = y * sh + ry * dh - pad;
          if (iy < 0 || iy >= H) continue;
          for (int rx = 0; rx < KW; ++rx) {
            const int ix = x * sw + rx * dw - pad;
            if (ix < 0 || ix >= W) continue;
            const size_t ibase = (((size_t)n * H + iy) * W + ix) * CI;
            const size_t wbase = ((size_t)ry * KW + rx) * CI * CO;
            for (int rc = 0; rc < CI; ++rc) {
              const double a = (double)half_to_float(in[ibase + rc]);
              for (int f = 0; f < CO; ++f)
                acc[f] += a * (double)half_to_float(w[wbase + (size_t)rc * CO + f]);
            }
          }
        }
        const size_t obase = (((size_t)n * HO + y) * WO + x) * CO;
        if (out_half) {
          uint16_t* o = (uint16_t*)out + obase;
          for (int f = 0; f < CO; ++f) o[f] = float_to_half_rn((float)acc[f]);
        } else {
          float* o = (float*)out + obase;
          for (int f = 0; f < CO; ++f) o[f] = (float)acc[f];
        }
      }
}

/*
 * NCHW conv, the operator of the reference's network tables (ops/cuda/conv2d.py:9-101), written
 * as the direct sum its im2col GEMM computes:
 *   out[n,c,p,q] = sum_{ci,kh,kw} pad(in)[n, ci, p*sh+kh, q*sw+kw] * w[c,ci,kh,kw]
 * `mode` 0: uint8/int8 operands (signedness flags), int32 output.  `mode` 1: binary16 operands,
 * double accumulation, float output; `mode` 2: the same rounded to binary16.
 */
void oracle_conv2d_nchw(const void* in, const void* w, void* out, int N, int H, int W, int CI, int CO,
                        int KH, int KW, int sh, int sw, int pad, int mode, int in_signed,
                        int w_signed) {
  const int HO = oracle_conv_out_extent(H, KH, sh, pad, 1);
  const int WO = oracle_conv_out_extent(W, KW, sw, pad, 1);
  for (int n = 0; n < N; ++n)
    for (int c = 0; c < CO; ++c)
      for (int p = 0; p < HO; ++p)
        for (int q = 0; q < WO; ++q) {
          int32_t iacc = 0;
          double facc = 0.0;
          for (int ci = 0; ci < CI; ++ci)
            for (int kh = 0; kh < KH; ++kh) {
              const int iy = p * sh + kh - pad;
              if (iy < 0 || iy >= H) continue;
              for (int kw = 0; kw < KW; ++kw) {
                const int ix = q * sw + kw - pad;
                if (ix < 0 || ix >= W) continue;
                const size_t ii = (((size_t)n * CI + ci) * H + iy) * W + ix;
                const size_t wi = (((size_t)c * CI + ci) * KH + kh) * KW + kw;
                if (mode == 0)
                  iacc += load_i8(in, ii, in_signed) * load_i8(w, wi, w_signed);
                else
                  facc += (double)half_to_float(((const uint16_t*)in)[ii]) *
                          (double)half_to_float(((const uint16_t*)w)[wi]);
              }
            }
          const size_t oi = (((size_t)n * CO + c) * HO + p) * WO + q;
          if (mode == 0) ((int32_t*)out)[oi] = iacc;
          else if (mode == 1) ((float*)out)[oi] = (float)facc;
          else ((uint16_t*)out)[oi] = float_to_half_rn((float)facc);
        }
}

/*
 * Tensor-core matrix-vector product, ops/cuda/gemv.py:12-30: the vector B (1,K) becomes an
 * (8,K) matrix whose rows 1..7 are zero; out[i,j] = sum_k A[i,k] * BPad[j,k], out (M,8).
 * `mode` 0: integer operands, int32 output; 1: binary16 operands, float output; 2: binary16 output.
 */
void oracle_gemv(const void* A, const void* x, void* out, int M, int K, int mode, int a_signed,
                 int x_signed) {
  for (int i = 0; i < M; ++i) {
    for (int j = 0; j < 8; ++j) {
      if (mode == 0) {
        int32_t acc = 0;
        for (int k = 0; k < K; ++k) {
          const int32_t b = (j == 0) ? load_i8(x, (size_t)k, x_signed) : 0;
          acc += load_i8(A, (size_t)i * K + k, a_signed) * b;
        }
        ((int32_t*)out)[(size_t)i * 8 + j] = acc;
      } else {
        double acc = 0.0;
        for (int k = 0; k < K; ++k) {
          const double b = (j == 0) ? (double)half_to_float(((const uint16_t*)x)[k]) : 0.0;
          acc += (double)half_to_float(((const uint16_t*)A)[(size_t)i * K + k]) * b;
        }
        if (mode == 1) ((float*)out)[(size_t)i * 8 + j] = (float)acc;
        else ((uint16_t*)out)[(size_t)i * 8 + j] = float_to_half_rn((float)acc);
      }
    }
  }
}

/*
 * NCW conv1d, ops/cuda/conv1d.py:23-69 written as the direct sum its im2col GEMM computes:
 *   out[n,c,q] = sum_{ci,kw} pad(in)[n, ci, q*stride + kw] * w[c,ci,kw],  W_O = (W - KW + 2*pad)/stride + 1
 * `pad` zeros on both ends of the width (get_pad_tuple1d of an int).  Modes as oracle_gemv.
 */
void oracle_conv1d_ncw(const void* in, const void* w, void* out, int N, int W, int CI, int CO, int KW,
                       int stride, int pad, int mode, int in_signed, int w_signed) {
  const int WO = (W - KW + 2 * pad) / stride + 1;
  for (int n = 0; n < N; ++n)
    for (int c = 0; c < CO; ++c)
      for (int q = 0; q < WO; ++q) {
        int32_t iacc = 0;
        double dacc = 0.0;
        for (int ci = 0; ci < CI; ++ci)
          for (int kw = 0; kw < KW; ++kw) {
            const int xw = q * stride + kw - pad;
            if (xw < 0 || xw >= W) continue;
            const size_t ii = ((size_t)n * CI + ci) * W + xw;
            const size_t wi = ((size_t)c * CI + ci) * KW + kw;
            if (mode == 0) iacc += load_i8(in, ii, in_signed) * load_i8(w, wi, w_signed);
            else dacc += (double)half_to_float(((const uint16_t*)in)[ii]) *
                         (double)half_to_float(((const uint16_t*)w)[wi]);
          }
        const size_t oi = ((size_t)n * CO + c) * WO + q;
        if (mode == 0) ((int32_t*)out)[oi] = iacc;
        else if (mode == 1) ((float*)out)[oi] = (float)dacc;
        else ((uint16_t*)out)[oi] = float_to_half_rn((float)dacc);
      }
}

/*
 * The DL Boost NWC conv1d, ops/x86/conv1d_int8.py:53-84: input uint8 (N,W,CI), filter int8
 * (CO/sco, KW, CI/4, sco, 4), output int32 (N, W_O, CO/sco, sco);
 *   out[n,x,oc,ob] = sum_{rx,icc,icb} pad(in)[n, x*stride + rx*dil, icc*4+icb] * w[oc,rx,icc,ob,icb]
 */
void oracle_conv1d_nwc_packed(const uint8_t* in, const int8_t* wp, int32_t* out, int N, int W, int CI,
                              int CO, int KW, int stride, int pad, int dil, int sco) {
  const int WO = (W - ((KW - 1) * dil + 1) + 2 * pad) / stride + 1;
  const int OC = CO / sco, IC = CI / 4;
  for (int n = 0; n < N; ++n)
    for (int x = 0; x < WO; ++x)
      for (int oc = 0; oc < OC; ++oc)
        for (int ob = 0; ob < sco; ++ob) {
          int32_t acc = 0;
          for (int rx = 0; rx < KW; ++rx) {
            const int xw = x * stride + rx * dil - pad;
            if (xw < 0 || xw >= W) continue;
            for (int icc = 0; icc < IC; ++icc)
              for (int icb = 0; icb < 4; ++icb) {
                const int32_t a = in[((size_t)n * W + xw) * CI + icc * 4 + icb];
                const int32_t b = wp[((((size_t)oc * KW + rx) * IC + icc) * sco + ob) * 4 + icb];
                acc += a * b;
              }
          }
          out[(((size_t)n * WO + x) * OC + oc) * sco + ob] = acc;
        }
}

/*
 * scan, ops/cuda/scan.py:6-23 and ops/x86/scan.py:11-27: out[i,j] = sum_k A[i,k] * B[j,k] with the
 * constant B[j,k] = (j <= k) ? 0 : 1.  `mode` 0: uint8/int8 A, int32 output; 1: binary16 A, float
 * output; 2: binary16 output.
 */
void oracle_scan(const void* A, void* out, int M, int N, int K, int mode, int a_signed) {
  for (int i = 0; i < M; ++i)
    for (int j = 0; j < N; ++j) {
      int32_t iacc = 0;
      double dacc = 0.0;
      for (int k = 0; k < K; ++k) {
        const int b = (j <= k) ? 0 : 1;
        if (mode == 0) iacc += load_i8(A, (size_t)i * K + k, a_signed) * b;
        else dacc += (double)half_to_float(((const uint16_t*)A)[(size_t)i * K + k]) * (double)b;
      }
      const size_t o = (size_t)i * N + j;
      if (mode == 0) ((int32_t*)out)[o] = iacc;
      else if (mode == 1) ((float*)out)[o] = (float)dacc;
      else ((uint16_t*)out)[o] = float_to_half_rn((float)dacc);
    }
}

/*
 * NCDHW conv3d, ops/cuda/conv3d.py:23-85 as the direct sum its im2col GEMM computes:
 *   out[n,c,d,p,q] = sum_{ci,kd,kh,kw} pad(in)[n,ci,d*sd+kd,p*sh+kh,q*sw+kw] * w[c,ci,kd,kh,kw]
 * `pad` zeros on every side of the three spatial axes.  Modes as oracle_conv1d_ncw.
 */
void oracle_conv3d_ncdhw(const void* in, const void* w, void* out, int N, int D, int H, int W, int CI,
                         int CO, int KD, int KH, int KW, int sd, int sh, int sw, int pad, int mode,
                         int in_signed, int w_signed) {
  const int DO = (D - KD + 2 * pad) / sd + 1, HO = (H - KH + 2 * pad) / sh + 1, WO = (W - KW + 2 * pad) / sw + 1;
  for (int n = 0; n < N; ++n)
    for (int c = 0; c < CO; ++c)
      for (int d = 0; d < DO; ++d)
        for (int p = 0; p < HO; ++p)
          for (int q = 0; q < WO; ++q) {
            int32_t iacc = 0;
            double dacc = 0.0;
            for (int ci = 0; ci < CI; ++ci)
              for (int kd = 0; kd < KD; ++kd) {
                const int z = d * sd + kd - pad;
                if (z < 0 || z >= D) continue;
                for (int kh = 0; kh < KH; ++kh) {
                  const int y = p * sh + kh - pad;
                  if (y < 0 || y >= H) continue;
                  for (int kw = 0; kw < KW; ++kw) {
                    const int x = q * sw + kw - pad;
                    if (x < 0 || x >= W) continue;
                    const size_t ii = ((((size_t)n * CI + ci) * D + z) * H + y) * W + x;
                    const size_t wi = ((((size_t)c * CI + ci) * KD + kd) * KH + kh) * KW + kw;
                    if (mode == 0) iacc += load_i8(in, ii, in_signed) * load_i8(w, wi, w_signed);
                    else dacc += (double)half_to_float(((const uint16_t*)in)[ii]) *
                                 (double)half_to_float(((const uint16_t*)w)[wi]);
                  }
                }
              }
            const size_t oi = ((((size_t)n * CO + c) * DO + d) * HO + p) * WO + q;
            if (mode == 0) ((int32_t*)out)[oi] = iacc;
            else if (mode == 1) ((float*)out)[oi] = (float)dacc;
            else ((uint16_t*)out)[oi] = float_to_half_rn((float)dacc);
          }
}
