// Small kernels around the MMA kernels: the scan operand, the x86 filter unpack, the layout
// glue of the NCHW operators (input / filter transposes, the few-channel form, the split-K
// reduction that writes NCHW).
#pragma once
#include "hb_kernel.cuh"

namespace hb {

// The constant operand of the reference's scan operator: B[i][j] = (i <= j) ? 0 : 1, an (N, K)
// matrix whose product with A gives out[m][n] = sum of A[m][k] over k < n.
template <typename T>
__global__ void hb_scan_mask_kernel(T* __restrict__ b, int N, int K, T one) {
  griddep_launch_dependents();
  const long long total = static_cast<long long>(N) * K;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int row = static_cast<int>(i / K), col = static_cast<int>(i - static_cast<long long>(row) * K);
    b[i] = row <= col ? T(0) : one;
  }
}

// Unpacks the x86 operator's int8 filter (CO/sco, KH, KW, CI/4, sco, 4) to HWIO (KH,KW,CI,CO).
// One thread per 4-byte group of input channels; consecutive threads walk output channels so
// that the HWIO writes of a warp land in consecutive bytes of four rows.
__global__ void hb_unpack_filter_kernel(const int8_t* __restrict__ packed, int8_t* __restrict__ hwio,
                                        int CO, int KH, int KW, int CI, int sco) {
  griddep_launch_dependents();
  const long long total = static_cast<long long>(KH) * KW * (CI / 4) * CO;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int co = static_cast<int>(i % CO);
    long long rest = i / CO;
    const int icc = static_cast<int>(rest % (CI / 4));
    rest /= (CI / 4);
    const int rx = static_cast<int>(rest % KW);
    const int ry = static_cast<int>(rest / KW);
    const int oc_chunk = co / sco, oc_block = co - oc_chunk * sco;
    const long long src =
        ((((static_cast<long long>(oc_chunk) * KH + ry) * KW + rx) * (CI / 4) + icc) * sco + oc_block) * 4;
    const int32_t four = *reinterpret_cast<const int32_t*>(packed + src);
    const long long dst0 = ((static_cast<long long>(ry) * KW + rx) * CI + icc * 4) * CO + co;
#pragma unroll
    for (int j = 0; j < 4; ++j)
      hwio[dst0 + static_cast<long long>(j) * CO] = static_cast<int8_t>((four >> (8 * j)) & 0xFF);
  }
}

// Layout glue of the NCHW operators in one launch: blocks [0, in_blocks) transpose the input
// (N, CI, P) to (N, P, CIp) with channels zero-padded to CIp, the rest bring the filter
// (CO, CI, T) to (T, CIp, CO).
constexpr int kFilterRun = 128;  // filter elements staged per output channel and block

struct NchwPre {
  const void* in; void* in_t;
  const void* w; void* w_t;
  int N, CI, CIp, P, CO, T;
  int vec, f_vec;                   // 8-byte accesses are possible (input; 1-tap filter)
  // strided 1x1 conv: only the pixels the conv reads are kept.  P counts kept pixels (HO*WO); kept
  // pixel j sits at source pixel (j / sub_wo) * sub_row + (j % sub_wo) * sub_col.  sub_wo = 0: all.
  int sub_wo, sub_col, sub_row, src_P;
  int in_bx, in_by, in_blocks;      // input tiles per image along P and along CIp; total
  int f_ci_tile, f_tchunk, f_bco, f_bci, f_bt;  // filter tiling (f_bco x f_bci tiles when T == 1)
};

// One (16*VEC)^2 tile of  dst[j*Rp + i] = (i < R && j < C) ? src[i*pitch + j] : 0,  i < Rp, j < Cp.
// 256 threads.  With `vec`, global accesses are 8 bytes wide: a warp reads 256 contiguous bytes of
// a source row and writes 128 contiguous bytes of a destination row per instruction.
template <typename T, int PITCH>
__device__ __forceinline__ void transpose_tile(T (*tile)[PITCH], const T* __restrict__ s, T* __restrict__ d,
                                               int R, int C, int Rp, int Cp, long long pitch, int i0,
                                               int j0, bool vec, int sub_wo = 0, int sub_col = 1,
                                               int sub_row = 0) {
  constexpr int VEC = 8 / sizeof(T);
  constexpr int TILE = 16 * VEC;
  const int tid = threadIdx.x;
  if (vec) {
    const int lane16 = tid & 15, grp = tid >> 4;
    uint2 v[VEC];  // TILE / 16 = VEC passes; all loads are issued before the first shared-memory store
#pragma unroll
    for (int u = 0; u < VEC; ++u) {
      const int i = i0 + grp + 16 * u, j = j0 + lane16 * VEC;
      v[u] = make_uint2(0u, 0u);
      if (i < R && j < C) v[u] = *reinterpret_cast<const uint2*>(s + i * pitch + j);
    }
#pragma unroll
    for (int u = 0; u < VEC; ++u) {
      uint32_t* t32 = reinterpret_cast<uint32_t*>(&tile[grp + 16 * u][lane16 * VEC]);
      t32[0] = v[u].x;
      t32[1] = v[u].y;
    }
    __syncthreads();
    for (int jj = grp; jj < TILE; jj += 16) {
      const int j = j0 + jj, i = i0 + lane16 * VEC;
      if (j >= Cp || i >= Rp) continue;
      __align__(8) T e[VEC];
#pragma unroll
      for (int r = 0; r < VEC; ++r) e[r] = tile[lane16 * VEC + r][jj];
      *reinterpret_cast<uint2*>(d + static_cast<long long>(j) * Rp + i) = *reinterpret_cast<const uint2*>(e);
    }
  } else {
    for (int base = tid; base < TILE * TILE; base += 4 * 256) {  // TILE * TILE is a multiple of 1024
      T v[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int idx = base + u * 256;
        const int ii = idx / TILE, jj = idx - ii * TILE;
        const int i = i0 + ii, j = j0 + jj;
        long long col = j;
        if (sub_wo > 0) {
          const int jy = j / sub_wo;
          col = static_cast<long long>(jy) * sub_row + (j - jy * sub_wo) * sub_col;
        }
        v[u] = (i < R && j < C) ? s[i * pitch + col] : T(0);
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int idx = base + u * 256;
        tile[idx / TILE][idx % TILE] = v[u];
      }
    }
    __syncthreads();
    for (int idx = tid; idx < TILE * TILE; idx += 256) {
      const int jj = idx / TILE, ii = idx - jj * TILE;
      const int i = i0 + ii, j = j0 + jj;
      if (j < Cp && i < Rp) d[static_cast<long long>(j) * Rp + i] = tile[ii][jj];
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(256) hb_nchw_pre_kernel(const NchwPre g) {
  constexpr int VEC = 8 / sizeof(T);
  constexpr int TILE = 16 * VEC;
  constexpr int PITCH = TILE + 4 / sizeof(T);   // row pitch of 33 words: conflict-free column reads
  constexpr int FPITCH = kFilterRun + 4 / sizeof(T);
  constexpr size_t kTileBytes = sizeof(T) * TILE * PITCH;
  constexpr size_t kFiltBytes = sizeof(T) * 32 * FPITCH;
  __shared__ __align__(8) uint8_t raw[kTileBytes > kFiltBytes ? kTileBytes : kFiltBytes];
  T (*tile)[PITCH] = reinterpret_cast<T (*)[PITCH]>(raw);
  griddep_launch_dependents();  // the conv kernel behind this one may set itself up meanwhile
  if (static_cast<int>(blockIdx.x) < g.in_blocks) {
    // ---- input: per image a (CI x P) matrix, transposed to (P x CIp) ----
    int b = blockIdx.x;
    const int bx = b % g.in_bx; b /= g.in_bx;   // along P
    const int by = b % g.in_by;                 // along CI
    const int n = b / g.in_by;
    const int src_P = g.sub_wo > 0 ? g.src_P : g.P;
    transpose_tile<T, PITCH>(tile, static_cast<const T*>(g.in) + static_cast<long long>(n) * g.CI * src_P,
                             static_cast<T*>(g.in_t) + static_cast<long long>(n) * g.P * g.CIp, g.CI, g.P,
                             g.CIp, g.P, src_P, by * TILE, bx * TILE, g.vec != 0, g.sub_wo, g.sub_col,
                             g.sub_row);
    return;
  }
  int b = blockIdx.x - g.in_blocks;
  if (g.T == 1) {
    // ---- one-tap filter: a (CO x CI) matrix, transposed to (CIp x CO) ----
    const int bci = b % g.f_bci, bco = b / g.f_bci;
    transpose_tile<T, PITCH>(tile, static_cast<const T*>(g.w), static_cast<T*>(g.w_t), g.CO, g.CI, g.CO,
                             g.CIp, g.CI, bco * TILE, bci * TILE, g.f_vec != 0);
    return;
  }
  // ---- filter with taps: 32 output channels x f_ci_tile input channels x f_tchunk taps per block.
  // For one output channel those source elements are one contiguous run (f_tchunk == T), or a run
  // of taps of a single input channel (T > kFilterRun).
  T (*fbuf)[FPITCH] = reinterpret_cast<T (*)[FPITCH]>(raw);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int bt = b % g.f_bt; b /= g.f_bt;
  const int bci = b % g.f_bci;
  const int bco = b / g.f_bci;
  const int co0 = bco * 32, ci0 = bci * g.f_ci_tile, t0 = bt * g.f_tchunk;
  const int nt = min(g.f_tchunk, g.T - t0);
  const int run = g.f_ci_tile * nt;
  const int run_valid = min(run, max(0, g.CI - ci0) * nt);  // beyond it: zero-padded channels
  const T* w = static_cast<const T*>(g.w);
  T* wt = static_cast<T*>(g.w_t);
  {
    T v[4][4];  // 16 independent loads per thread: the loop is bound by load latency otherwise
#pragma unroll
    for (int cc = 0; cc < 4; ++cc) {
      const int co = co0 + warp + 8 * cc;
      const T* srow = w + (static_cast<long long>(co) * g.CI + ci0) * g.T + t0;
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int r = lane + 32 * u;
        v[cc][u] = (co < g.CO && r < run_valid) ? srow[r] : T(0);
      }
    }
#pragma unroll
    for (int cc = 0; cc < 4; ++cc)
#pragma unroll
      for (int u = 0; u < 4; ++u)
        if (lane + 32 * u < run) fbuf[warp + 8 * cc][lane + 32 * u] = v[cc][u];
  }
  __syncthreads();
  const int co = co0 + lane;
  for (int r = warp; r < run; r += 8) {
    const int cil = r / nt;
    const int ci = ci0 + cil, t = t0 + (r - cil * nt);
    if (co < g.CO && ci < g.CIp) wt[(static_cast<long long>(t) * g.CIp + ci) * g.CO + co] = fbuf[lane][r];
  }
}

// Last step of a split-K NCHW conv: sums the `slabs` partial results ws[s][n*P + pix][co] in slab
// order and writes out[n][co][pix].  32 x 32 tiles through shared memory: reads coalesced along
// co, writes along pix.
template <typename ACC, typename OUT>
__global__ void hb_nchw_post_kernel(const ACC* __restrict__ ws, OUT* __restrict__ out, int slabs,
                                    long long slab_elems, int P, int CO) {
  __shared__ ACC tile[32][33];
  const int n = blockIdx.z, p0 = blockIdx.x * 32, c0 = blockIdx.y * 32;
  for (int pp = threadIdx.y; pp < 32; pp += blockDim.y) {
    const int pix = p0 + pp, co = c0 + threadIdx.x;
    ACC acc = ACC(0);
    if (pix < P && co < CO) {
      const ACC* src = ws + (static_cast<long long>(n) * P + pix) * CO + co;
      for (int s = 0; s < slabs; ++s) acc += src[s * slab_elems];
    }
    tile[pp][threadIdx.x] = acc;
  }
  __syncthreads();
  for (int cc = threadIdx.y; cc < 32; cc += blockDim.y) {
    const int co = c0 + cc, pix = p0 + threadIdx.x;
    if (co < CO && pix < P) out[(static_cast<long long>(n) * CO + co) * P + pix] = static_cast<OUT>(tile[threadIdx.x][cc]);
  }
}

// Layout glue of an NCHW conv with very few input channels (the first layer of an image
// network).  The input becomes a zero-bordered (N, Hs, Ws, cis) tensor with cis = 16 bytes of
// channels per pixel; the conv kernel then reads, as one "pixel" of KWp * cis channels, KWp
// horizontally adjacent pixels at once (a tensor map whose W stride is one real pixel), so a
// whole filter row is one K block.  The filter (CO, CI, KH, KW) becomes (KH, KWp, cis, CO) with
// zeros for the padded taps and channels.
struct StemPre {
  const void* in; void* in_t;
  const void* w; void* w_t;
  int N, CI, H, W, CO, KH, KW, KWp, cis, Hs, Ws, pad_h, pad_w;
  long long in_px, w_elems;
};

template <typename T>
__global__ void __launch_bounds__(256) hb_nchw_stem_pre_kernel(const StemPre g) {
  constexpr int CIS = 16 / sizeof(T);
  griddep_launch_dependents();  // the conv kernel behind this one may set itself up meanwhile
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  const long long first = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
  const T* in = static_cast<const T*>(g.in);
  for (long long idx = first; idx < g.in_px; idx += stride) {
    const int ws = static_cast<int>(idx % g.Ws);
    const long long rest = idx / g.Ws;
    const int hs = static_cast<int>(rest % g.Hs);
    const int n = static_cast<int>(rest / g.Hs);
    const int y = hs - g.pad_h, x = ws - g.pad_w;
    __align__(16) T v[CIS];
#pragma unroll
    for (int c = 0; c < CIS; ++c) v[c] = T(0);
    if (y >= 0 && y < g.H && x >= 0 && x < g.W) {
#pragma unroll
      for (int c = 0; c < CIS; ++c)
        if (c < g.CI) v[c] = in[((static_cast<long long>(n) * g.CI + c) * g.H + y) * g.W + x];
    }
    reinterpret_cast<uint4*>(g.in_t)[idx] = *reinterpret_cast<const uint4*>(v);
  }
  const T* w = static_cast<const T*>(g.w);
  T* wt = static_cast<T*>(g.w_t);
  for (long long idx = first; idx < g.w_elems; idx += stride) {
    const int co = static_cast<int>(idx % g.CO);
    long long r = idx / g.CO;
    const int ci = static_cast<int>(r % CIS); r /= CIS;
    const int kw = static_cast<int>(r % g.KWp);
    const int kh = static_cast<int>(r / g.KWp);
    wt[idx] = (ci < g.CI && kw < g.KW)
                  ? w[((static_cast<long long>(co) * g.CI + ci) * g.KH + kh) * g.KW + kw] : T(0);
  }
}

}  // namespace hb
