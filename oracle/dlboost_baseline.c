/*
 * dlboost_baseline.c — the timed CPU baseline.  TEST / BENCHMARK INFRASTRUCTURE ONLY.
 *
 * A C port of the structure of the reference's tuned x86 ("DL Boost") programs, which TVM would
 * generate and which cannot be generated here: an OpenMP `parallel for` over fused outer spatial
 * tiles (schedule/sched_op/cpu_operator.py:17-27), an output tile kept in registers / L1
 * (the cache-write stage of ops/x86/dense.py:23), and the 16-lane x 4-deep AVX512-VNNI
 * `vpdpbusd` micro-kernel the operators name (dot_16x1x16_uint8_int8_int32_cascadelake,
 * ops/x86/dense.py:25, applied at cpu_operator.py:84-117).  Conv takes the x86 operator's own
 * packed filter (CO/sco,KH,KW,CI/4,sco,4) (ops/x86/conv2d_int8.py:36-50).
 *
 * The fp16 operators have no x86 path in the reference (ops/x86 is int8 only); the fp32 GEMM
 * and conv here are the CPU column for those configurations, labelled as a port.
 *
 * Every kernel has a scalar twin chosen at run time when the CPU lacks AVX512-VNNI.  Results
 * are exact for the integer kernels and are checked against heron_oracle.c by the tests.
 */
#include <immintrin.h>
#include <omp.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define VNNI_TARGET __attribute__((target("avx512f,avx512bw,avx512vl,avx512vnni")))
#define AVX512_TARGET __attribute__((target("avx512f,avx512bw,avx512vl,f16c")))

int dlb_has_vnni(void) {
  __builtin_cpu_init();
  return __builtin_cpu_supports("avx512vnni") && __builtin_cpu_supports("avx512f");
}
int dlb_has_avx512(void) {
  __builtin_cpu_init();
  return __builtin_cpu_supports("avx512f");
}
int dlb_max_threads(void) { return omp_get_max_threads(); }
void dlb_set_threads(int n) { if (n > 0) omp_set_num_threads(n); }

/* Packs B (N,K) int8 into [N/16][K/4][16][4]: the operand order vpdpbusd wants. */
static void pack_b_16x4(const int8_t* B, int8_t* P, int N, int K) {
  const int NB = N / 16, KB = K / 4;
#pragma omp parallel for schedule(static)
  for (int nb = 0; nb < NB; ++nb)
    for (int kb = 0; kb < KB; ++kb)
      for (int j = 0; j < 16; ++j)
        memcpy(P + ((((size_t)nb * KB + kb) * 16 + j) * 4), B + (size_t)(nb * 16 + j) * K + kb * 4, 4);
}

VNNI_TARGET static void gemm_u8s8_vnni_tile(const uint8_t* A, const int8_t* P, int32_t* C, int M,
                                            int K, int N, int i0, int nb) {
  /* 4 rows x 16 columns of C per register tile. */
  const int KB = K / 4;
  const int8_t* p = P + (size_t)nb * KB * 64;
  int rows = M - i0 < 4 ? M - i0 : 4;
  __m512i acc0 = _mm512_setzero_si512(), acc1 = acc0, acc2 = acc0, acc3 = acc0;
  const uint8_t* a0 = A + (size_t)i0 * K;
  const uint8_t* a1 = a0 + (rows > 1 ? K : 0);
  const uint8_t* a2 = a0 + (rows > 2 ? 2 * (size_t)K : 0);
  const uint8_t* a3 = a0 + (rows > 3 ? 3 * (size_t)K : 0);
  for (int kb = 0; kb < KB; ++kb) {
    const __m512i b = _mm512_loadu_si512((const void*)(p + (size_t)kb * 64));
    int32_t w0, w1, w2, w3;
    memcpy(&w0, a0 + kb * 4, 4); memcpy(&w1, a1 + kb * 4, 4);
    memcpy(&w2, a2 + kb * 4, 4); memcpy(&w3, a3 + kb * 4, 4);
    acc0 = _mm512_dpbusd_epi32(acc0, _mm512_set1_epi32(w0), b);
    acc1 = _mm512_dpbusd_epi32(acc1, _mm512_set1_epi32(w1), b);
    acc2 = _mm512_dpbusd_epi32(acc2, _mm512_set1_epi32(w2), b);
    acc3 = _mm512_dpbusd_epi32(acc3, _mm512_set1_epi32(w3), b);
  }
  int32_t* c = C + (size_t)i0 * N + nb * 16;
  _mm512_storeu_si512((void*)c, acc0);
  if (rows > 1) _mm512_storeu_si512((void*)(c + N), acc1);
  if (rows > 2) _mm512_storeu_si512((void*)(c + 2 * (size_t)N), acc2);
  if (rows > 3) _mm512_storeu_si512((void*)(c + 3 * (size_t)N), acc3);
}

static void gemm_u8s8_scalar(const uint8_t* A, const int8_t* B, int32_t* C, int M, int K, int N) {
#pragma omp parallel for schedule(static)
  for (int i = 0; i < M; ++i)
    for (int j = 0; j < N; ++j) {
      int32_t acc = 0;
      for (int k = 0; k < K; ++k) acc += (int32_t)A[(size_t)i * K + k] * (int32_t)B[(size_t)j * K + k];
      C[(size_t)i * N + j] = acc;
    }
}

/*
 * u8 (M,K) x s8 (N,K) -> s32 (M,N).  `pack` is scratch of N*K bytes (caller-owned); packing B is
 * part of the call, as the strided 16x4 reads are part of the reference's generated loop nest.
 * Needs N % 16 == 0 and K % 4 == 0 for the VNNI path; anything else runs the scalar twin.
 */
void dlb_gemm_u8s8(const uint8_t* A, const int8_t* B, int32_t* C, int M, int K, int N, int8_t* pack) {
  if (!dlb_has_vnni() || N % 16 != 0 || K % 4 != 0 || pack == NULL) {
    gemm_u8s8_scalar(A, B, C, M, K, N);
    return;
  }
  pack_b_16x4(B, pack, N, K);
  const int MB = (M + 3) / 4, NB = N / 16;
#pragma omp parallel for collapse(2) schedule(static)
  for (int mb = 0; mb < MB; ++mb)
    for (int nb = 0; nb < NB; ++nb) gemm_u8s8_vnni_tile(A, pack, C, M, K, N, mb * 4, nb);
}

/*
 * Batched s8 x s8 -> s32.  The reference's x86 batched operator is u8 x s8
 * (ops/x86/batch_matmul.py:9-10); a signed A is handled the way VNNI code does it: bias A by
 * +128 into u8, then subtract 128 * sum_k B[j,k] from every output column.
 * `a_bias` (batch*M*K bytes), `pack` (N*K bytes) and `colsum` (N int32) are caller-owned scratch.
 */
void dlb_bmm_s8s8(const int8_t* A, const int8_t* B, int32_t* C, int batch, int M, int K, int N,
                  uint8_t* a_bias, int8_t* pack, int32_t* colsum) {
  const size_t an = (size_t)batch * M * K;
#pragma omp parallel for schedule(static)
  for (size_t i = 0; i < an; ++i) a_bias[i] = (uint8_t)((int)A[i] + 128);
  for (int b = 0; b < batch; ++b) {
    const int8_t* Bb = B + (size_t)b * N * K;
    int32_t* Cb = C + (size_t)b * M * N;
    dlb_gemm_u8s8(a_bias + (size_t)b * M * K, Bb, Cb, M, K, N, pack);
#pragma omp parallel for schedule(static)
    for (int j = 0; j < N; ++j) {
      int32_t s = 0;
      for (int k = 0; k < K; ++k) s += Bb[(size_t)j * K + k];
      colsum[j] = 128 * s;
    }
#pragma omp parallel for schedule(static)
    for (int i = 0; i < M; ++i)
      for (int j = 0; j < N; ++j) Cb[(size_t)i * N + j] -= colsum[j];
  }
}

void dlb_bmm_u8s8(const uint8_t* A, const int8_t* B, int32_t* C, int batch, int M, int K, int N,
                  int8_t* pack) {
  for (int b = 0; b < batch; ++b)
    dlb_gemm_u8s8(A + (size_t)b * M * K, B + (size_t)b * N * K, C + (size_t)b * M * N, M, K, N, pack);
}

/* ---- conv, x86 operator layout ------------------------------------------------------------ */
static int out_extent(int in, int k, int stride, int pad, int dil) {
  return (in - ((k - 1) * dil + 1) + 2 * pad) / stride + 1;
}

VNNI_TARGET static void conv_pixel_vnni(const uint8_t* in, const int8_t* wp, int32_t* o, int H, int W,
                                        int CI, int KH, int KW, int n, int y, int x, int sh, int sw,
                                        int pad, int dh, int dw, int sco, int occ) {
  /* One output pixel, one chunk of `sco` output channels (sco/16 vectors). */
  const int nv = sco / 16, ICC = CI / 4;
  __m512i acc[4];
  for (int v = 0; v < nv; ++v) acc[v] = _mm512_setzero_si512();
  for (int ry = 0; ry < KH; ++ry) {
    const int iy = y * sh + ry * dh - pad;
    if (iy < 0 || iy >= H) continue;
    for (int rx = 0; rx < KW; ++rx) {
      const int ix = x * sw + rx * dw - pad;
      if (ix < 0 || ix >= W) continue;
      const uint8_t* a = in + (((size_t)n * H + iy) * W + ix) * CI;
      const int8_t* wrow = wp + ((((size_t)occ * KH + ry) * KW + rx) * ICC) * sco * 4;
      for (int icc = 0; icc < ICC; ++icc) {
        int32_t w4;
        memcpy(&w4, a + icc * 4, 4);
        const __m512i av = _mm512_set1_epi32(w4);
        const int8_t* wv = wrow + (size_t)icc * sco * 4;
        for (int v = 0; v < nv; ++v)
          acc[v] = _mm512_dpbusd_epi32(acc[v], av, _mm512_loadu_si512((const void*)(wv + v * 64)));
      }
    }
  }
  for (int v = 0; v < nv; ++v) _mm512_storeu_si512((void*)(o + v * 16), acc[v]);
}

static void conv_pixel_scalar(const uint8_t* in, const int8_t* wp, int32_t* o, int H, int W, int CI,
                              int KH, int KW, int n, int y, int x, int sh, int sw, int pad, int dh,
                              int dw, int sco, int occ) {
  const int ICC = CI / 4;
  for (int ocb = 0; ocb < sco; ++ocb) o[ocb] = 0;
  for (int ry = 0; ry < KH; ++ry) {
    const int iy = y * sh + ry * dh - pad;
    if (iy < 0 || iy >= H) continue;
    for (int rx = 0; rx < KW; ++rx) {
      const int ix = x * sw + rx * dw - pad;
      if (ix < 0 || ix >= W) continue;
      const uint8_t* a = in + (((size_t)n * H + iy) * W + ix) * CI;
      const int8_t* wrow = wp + ((((size_t)occ * KH + ry) * KW + rx) * ICC) * sco * 4;
      for (int icc = 0; icc < ICC; ++icc)
        for (int ocb = 0; ocb < sco; ++ocb)
          for (int icb = 0; icb < 4; ++icb)
            o[ocb] += (int32_t)a[icc * 4 + icb] * (int32_t)wrow[((size_t)icc * sco + ocb) * 4 + icb];
    }
  }
}

/*
 * u8 NHWC input, packed s8 filter (CO/sco,KH,KW,CI/4,sco,4), s32 output (N,HO,WO,CO/sco,sco).
 * Parallel over the fused (n, y, x, oc_chunk) loop, as the reference's schedule does.
 */
void dlb_conv2d_nhwc_packed(const uint8_t* in, const int8_t* wp, int32_t* out, int N, int H, int W,
                            int CI, int CO, int KH, int KW, int sh, int sw, int pad, int dh, int dw,
                            int sco) {
  const int HO = out_extent(H, KH, sh, pad, dh), WO = out_extent(W, KW, sw, pad, dw);
  const int OCC = CO / sco;
  const int vnni = dlb_has_vnni() && sco % 16 == 0 && sco <= 64 && CI % 4 == 0;
  const long long total = (long long)N * HO * WO * OCC;
#pragma omp parallel for schedule(static)
  for (long long t = 0; t < total; ++t) {
    const int occ = (int)(t % OCC);
    long long r = t / OCC;
    const int x = (int)(r % WO); r /= WO;
    const int y = (int)(r % HO);
    const int n = (int)(r / HO);
    int32_t* o = out + (size_t)t * sco;
    if (vnni)
      conv_pixel_vnni(in, wp, o, H, W, CI, KH, KW, n, y, x, sh, sw, pad, dh, dw, sco, occ);
    else
      conv_pixel_scalar(in, wp, o, H, W, CI, KH, KW, n, y, x, sh, sw, pad, dh, dw, sco, occ);
  }
}

/* ---- fp32 port for the fp16 configurations ------------------------------------------------ */
AVX512_TARGET static void widen_f16(const uint16_t* src, float* dst, size_t n) {
#pragma omp parallel for schedule(static)
  for (long long i = 0; i < (long long)(n / 16); ++i)
    _mm512_storeu_ps(dst + i * 16, _mm512_cvtph_ps(_mm256_loadu_si256((const __m256i*)(src + i * 16))));
  for (size_t i = n - n % 16; i < n; ++i) {
    const __m128i h = _mm_cvtsi32_si128(src[i]);
    dst[i] = _mm_cvtss_f32(_mm_cvtph_ps(h));
  }
}

AVX512_TARGET static void sgemm_nt_tile(const float* A, const float* B, float* C, int K, int N,
                                        int i0, int j0, int mi, int nj) {
  /* up to 4 x 4 outputs, each a 16-lane partial sum over K, reduced at the end */
  __m512 acc[4][4];
  for (int i = 0; i < 4; ++i)
    for (int j = 0; j < 4; ++j) acc[i][j] = _mm512_setzero_ps();
  const int K16 = K & ~15;
  for (int k = 0; k < K16; k += 16) {
    __m512 a[4], b[4];
    for (int i = 0; i < 4; ++i) a[i] = _mm512_loadu_ps(A + (size_t)(i0 + (i < mi ? i : 0)) * K + k);
    for (int j = 0; j < 4; ++j) b[j] = _mm512_loadu_ps(B + (size_t)(j0 + (j < nj ? j : 0)) * K + k);
    for (int i = 0; i < 4; ++i)
      for (int j = 0; j < 4; ++j) acc[i][j] = _mm512_fmadd_ps(a[i], b[j], acc[i][j]);
  }
  for (int i = 0; i < mi; ++i)
    for (int j = 0; j < nj; ++j) {
      float s = _mm512_reduce_add_ps(acc[i][j]);
      for (int k = K16; k < K; ++k) s += A[(size_t)(i0 + i) * K + k] * B[(size_t)(j0 + j) * K + k];
      C[(size_t)(i0 + i) * N + j0 + j] = s;
    }
}

/*
 * fp16 (M,K) x fp16 (N,K) -> fp32 (M,N): widen once to fp32 (scratch a32: M*K floats, b32: N*K
 * floats, caller-owned), then a register-tiled AVX512 FMA loop, parallel over output tiles.
 */
void dlb_gemm_f16(const uint16_t* A, const uint16_t* B, float* C, int M, int K, int N, float* a32,
                  float* b32) {
  if (!dlb_has_avx512()) return;
  widen_f16(A, a32, (size_t)M * K);
  widen_f16(B, b32, (size_t)N * K);
  const int MB = (M + 3) / 4, NB = (N + 3) / 4;
#pragma omp parallel for collapse(2) schedule(static)
  for (int mb = 0; mb < MB; ++mb)
    for (int nb = 0; nb < NB; ++nb) {
      const int mi = M - mb * 4 < 4 ? M - mb * 4 : 4, nj = N - nb * 4 < 4 ? N - nb * 4 : 4;
      sgemm_nt_tile(a32, b32, C, K, N, mb * 4, nb * 4, mi, nj);
    }
}
