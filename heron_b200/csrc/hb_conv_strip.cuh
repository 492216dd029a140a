// Stride-1 NHWC conv2d with a resident filter and halo strips ("strip" algorithm).
//
// The implicit-GEMM kernel fetches every input pixel once per filter tap.  For convolutions
// with few channels on large images (ResNet stage-2: 56x56x64, 3x3) that is nine L2 reads per
// pixel for a kernel whose floor is one HBM read.  Here a CTA instead
//   * keeps the whole HWIO filter in shared memory for the life of the kernel (it is loaded once
//     per CTA: KH*KW*CI*CO elements, 72 KiB for 3x3x64x64 fp16), and
//   * loads, per tile, one zero-padded strip of the input — (R + (KH-1)*dil) rows of the padded
//     width Wp = W + 2*pad_w — with a single tiled TMA box per 128-byte channel chunk; padding comes
//     from TMA's out-of-bounds zero fill (the box starts at w = -pad_w, h = y0 - pad_h).
// Output positions are numbered in padded-linear order i = y*Wp + x (x < Wp, so each row carries
// Wp - WO junk positions).  For filter tap (ry, rx) the A operand of the MMA is the same strip
// read from pixel (ry*dil*Wp + rx*dil) on: its shared-memory descriptor simply starts that many
// 128-byte rows into the strip.  The 128-byte swizzle is a function of the absolute shared-memory
// address, so a descriptor may start at any 128-byte row.  One tile = R = floor(128 / Wp) output
// rows of one image = one 128-row MMA per (tap, 32 bytes of channels).
//
// Roles as in hb_umma_kernel: warp 0 loads (filter once, then strips into a ring of two to six buffers),
// warp 1 issues MMAs into one of two TMEM accumulators, warps 2..5 read the accumulator and store
// the valid positions straight to global memory (each thread owns one output pixel: CO
// contiguous elements).  All waits are bounded, with the same abort protocol.
#pragma once
#include "hb_kernel.cuh"

namespace hb {

constexpr int kMaxStripRing = 6;

struct StripParams {
  int N, H, W, CI, CO, KH, KW, pad_h, pad_w, dil_h, dil_w, HO, WO;
  int Wp;             // padded width
  int R;              // output rows per tile
  int strip_rows;     // input rows per strip = R + (KH-1)*dil_h
  int strip_bytes;    // bytes reserved per channel chunk of a strip (multiple of 1024)
  int n_cchunks;      // 128-byte channel chunks per pixel
  int groups;         // tiles per image = ceil(HO / R)
  int num_tiles;
  int esize_in, esize_out;
  int tmem_cols;
  int ring;   // strip buffers in flight (2..kMaxStripRing)
  long long wait_limit_cycles;
  int probe;  // diagnostic modes of -DHB_PROBES builds: 2 = no MMAs, 3 = the epilogue only hands the accumulator
              // back, 4 = strips loaded once, 9 = the tile's MMAs on fixed descriptors (and 3)
  uint32_t idesc;
  void* out;
  int out_nchw;  // output is (N, CO, HO, WO) instead of (N, HO, WO, CO)
};

struct StripBars {
  uint64_t filt_full;
  uint64_t strip_full[kMaxStripRing];
  uint64_t strip_empty[kMaxStripRing];
  uint64_t tmem_full[2];
  uint64_t tmem_empty[2];
  uint64_t drain;
  uint32_t tmem_base;
  int abort_flag;
};

// Tiled 4-D load (c, w, h, n); w and h may be negative or past the end: those pixels read zero.
__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap* m, uint32_t bar, int c,
                                            int w, int h, int n) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5, %6}], [%2];" ::"r"(dst),
      "l"(reinterpret_cast<uint64_t>(m)), "r"(bar), "r"(c), "r"(w), "r"(h), "r"(n)
      : "memory");
}

template <int OUT_BYTES, int KIND>
__global__ void __launch_bounds__(kThreads, 1)
hb_conv_strip_kernel(const __grid_constant__ CUtensorMap tmIn, const __grid_constant__ CUtensorMap tmW,
                     const StripParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (smem_base - smem_u32(smem_raw));

  const int BK = 128 / p.esize_in;              // channels per 128-byte chunk
  const int tap_bytes = BK * p.CO * p.esize_in;  // one (tap, channel chunk) slab of the filter
  const int n_taps = p.KH * p.KW;
  const int filt_bytes = n_taps * p.n_cchunks * tap_bytes;
  const int strip_total = p.n_cchunks * p.strip_bytes;
  const uint32_t sFilt = smem_base;
  const uint32_t sStrip = sFilt + ((filt_bytes + 1023) & ~1023);
  StripBars* bars = reinterpret_cast<StripBars*>(smem + (sStrip - smem_base) + p.ring * strip_total);
  volatile int* abort_flag = &bars->abort_flag;
  const WaitCtx wctx{abort_flag, p.wait_limit_cycles > 0 ? p.wait_limit_cycles : HB_WAIT_LIMIT_CYCLES};

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    mbar_init(smem_u32(&bars->filt_full), 1);
    static_assert(sizeof(bars->strip_full) == kMaxStripRing * sizeof(uint64_t) &&
                      sizeof(bars->strip_empty) == kMaxStripRing * sizeof(uint64_t),
                  "every ring barrier below is initialised");
    for (int i = 0; i < kMaxStripRing; ++i) {
      mbar_init(smem_u32(&bars->strip_full[i]), 1);
      mbar_init(smem_u32(&bars->strip_empty[i]), 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(smem_u32(&bars->tmem_full[i]), 1);
      mbar_init(smem_u32(&bars->tmem_empty[i]), kEpiWarps);
    }
    mbar_init(smem_u32(&bars->drain), 1);
    bars->abort_flag = 0;
    fence_mbar_init();
    prefetch_tmap(&tmIn);
    prefetch_tmap(&tmW);
  }
  if (warp == 1) tmem_alloc_cg<1>(smem_u32(&bars->tmem_base), static_cast<uint32_t>(p.tmem_cols));
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = bars->tmem_base;
  griddep_wait();  // input and filter may come from a layout kernel this one was launched behind
  griddep_launch_dependents();  // the next launch of the stream may set itself up meanwhile

  if (warp == 0) {
    // ------------------------------ producer ----------------------------------------------
    if (elect_one()) {
      bool ok = true;
      // the filter, once: per (tap, channel chunk) one MN-major slab of BK rows x CO columns,
      // fetched as CO*esize/128 boxes of 128 bytes of output channels
      const int chunk_cols = 128 / p.esize_in;
      const int n_nchunks = p.CO / chunk_cols;
      const uint32_t ff = smem_u32(&bars->filt_full);
      mbar_arrive_expect_tx(ff, static_cast<uint32_t>(filt_bytes));
      for (int tap = 0; tap < n_taps; ++tap)
        for (int cc = 0; cc < p.n_cchunks; ++cc)
          for (int j = 0; j < n_nchunks; ++j)
            tma_load_3d(sFilt + (tap * p.n_cchunks + cc) * tap_bytes + j * (BK * 128), &tmW, ff,
                        j * chunk_cols, tap * p.CI + cc * BK, 0);
      int buf = 0;
      uint32_t phase = 0;
      int issued = 0;
      const uint32_t tx = static_cast<uint32_t>(p.n_cchunks * p.strip_rows * p.Wp * 128);
      for (int t = blockIdx.x; ok && t < p.num_tiles; t += gridDim.x) {
        const int n = t / p.groups;
        const int y0 = (t - n * p.groups) * p.R;
        if (!mbar_wait(smem_u32(&bars->strip_empty[buf]), phase ^ 1u, wctx)) {
          ok = false;
          break;
        }
        const uint32_t full = smem_u32(&bars->strip_full[buf]);
#ifdef HB_PROBES
        if (p.probe == 4 && issued >= p.ring) {
          mbar_arrive(full);
          ++issued;
          if (++buf == p.ring) {
            buf = 0;
            phase ^= 1u;
          }
          continue;
        }
#endif
        mbar_arrive_expect_tx(full, tx);
        for (int cc = 0; cc < p.n_cchunks; ++cc)
          tma_load_4d(sStrip + buf * strip_total + cc * p.strip_bytes, &tmIn, full, cc * BK, -p.pad_w,
                      y0 - p.pad_h, n);
        ++issued;
        if (++buf == p.ring) {
          buf = 0;
          phase ^= 1u;
        }
      }
      if (!ok) {
        mbar_wait_drain(smem_u32(&bars->filt_full), 0u);
        const int pending = issued < p.ring ? issued : p.ring;
        for (int i = 0; i < pending; ++i) {
          if (--buf < 0) {
            buf = p.ring - 1;
            phase ^= 1u;
          }
          mbar_wait_drain(smem_u32(&bars->strip_full[buf]), phase);
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------ MMA issuer --------------------------------------------
    if (elect_one()) {
      bool ok = mbar_wait(smem_u32(&bars->filt_full), 0u, wctx);
      int buf = 0, acc = 0;
      uint32_t phase = 0, acc_phase = 0;
      const int umma_k = 32 / p.esize_in;
      // A: K-major rows of 128 bytes, 8-row groups 1024 bytes apart.  B: MN-major, 128-byte
      // rows of output channels, 8-row groups 1024 bytes apart, column chunks BK*128 bytes apart.
      const uint64_t desc_hi = static_cast<uint64_t>((1024u >> 4) | (1u << 14) | (2u << 29)) << 32;
      const uint32_t a_lo_fixed = (16u >> 4) << 16;
      const uint32_t b_lo_fixed = ((static_cast<uint32_t>(BK * 128) >> 4) & 0x3FFFu) << 16;
      const uint32_t b_step16 = static_cast<uint32_t>(umma_k * 128) >> 4;
      const uint32_t idesc = p.idesc;
      for (int t = blockIdx.x; ok && t < p.num_tiles; t += gridDim.x) {
        if (!mbar_wait(smem_u32(&bars->tmem_empty[acc]), acc_phase ^ 1u, wctx) ||
            !mbar_wait(smem_u32(&bars->strip_full[buf]), phase, wctx)) {
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc * p.CO);
        uint32_t accum = 0u;
#ifdef HB_PROBES
        if (p.probe == 9) {
          // diagnostic: the tile's MMA count on fixed descriptors, no address arithmetic in the loop
          const uint32_t a_lo = (((sStrip + buf * strip_total) >> 4) & 0x3FFFu) | a_lo_fixed;
          const uint32_t b_lo = ((sFilt >> 4) & 0x3FFFu) | b_lo_fixed;
          const uint64_t da = desc_hi | a_lo, db = desc_hi | b_lo;
          const int n = p.KH * p.KW * p.n_cchunks * 4;
          umma_cg<1, KIND>(d_tmem, da, db, idesc, 0u);
#pragma unroll 4
          for (int i = 1; i < n; ++i) umma_cg<1, KIND>(d_tmem, da, db, idesc, 1u);
        } else if (p.probe != 2)
#endif
        for (int ry = 0; ry < p.KH; ++ry)
          for (int rx = 0; rx < p.KW; ++rx) {
            const uint32_t row_off = static_cast<uint32_t>(ry * p.dil_h * p.Wp + rx * p.dil_w) * 128u;
            for (int cc = 0; cc < p.n_cchunks; ++cc) {
              const uint32_t a_addr = sStrip + buf * strip_total + cc * p.strip_bytes + row_off;
              const uint32_t b_addr = sFilt + ((ry * p.KW + rx) * p.n_cchunks + cc) * tap_bytes;
              const uint32_t a_lo = ((a_addr >> 4) & 0x3FFFu) | a_lo_fixed;
              const uint32_t b_lo = ((b_addr >> 4) & 0x3FFFu) | b_lo_fixed;
#pragma unroll
              for (int k = 0; k < 4; ++k) {
                umma_cg<1, KIND>(d_tmem, desc_hi | (a_lo + 2u * k), desc_hi | (b_lo + b_step16 * k), idesc,
                                 accum);
                accum = 1u;
              }
            }
          }
        umma_commit(smem_u32(&bars->strip_empty[buf]));
        umma_commit(smem_u32(&bars->tmem_full[acc]));
        if (++buf == p.ring) {
          buf = 0;
          phase ^= 1u;
        }
        if (++acc == 2) {
          acc = 0;
          acc_phase ^= 1u;
        }
      }
      if (!ok) {
        umma_commit(smem_u32(&bars->drain));
        mbar_wait_drain(smem_u32(&bars->drain), 0u);
      }
    }
    __syncwarp();
  } else {
    // ------------------------------ epilogue ----------------------------------------------
    const int q = warp & 3;
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    constexpr int kColsPerStep = 128 / OUT_BYTES;  // 32 or 64 output channels = 128 bytes
    const int pos = q * 32 + lane;                 // padded-linear position inside the tile
    const int py = pos / p.Wp;
    const int px = pos - py * p.Wp;
    for (int t = blockIdx.x; ok && t < p.num_tiles; t += gridDim.x) {
      const int n = t / p.groups;
      const int y = (t - n * p.groups) * p.R + py;
      const bool valid = py < p.R && y < p.HO && px < p.WO;
      if (!mbar_wait(smem_u32(&bars->tmem_full[acc]), acc_phase, wctx)) {
        ok = false;
        break;
      }
      tc_fence_after();
      const uint32_t t_addr =
          tmem_base + (static_cast<uint32_t>(q * 32) << 16) + static_cast<uint32_t>(acc * p.CO);
      uint8_t* orow = static_cast<uint8_t*>(p.out) +
                      ((static_cast<long long>(n) * p.HO + y) * p.WO + px) * p.CO * OUT_BYTES;
#ifdef HB_PROBES
      if (p.probe == 3 || p.probe == 9) {
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&bars->tmem_empty[acc]));
        if (++acc == 2) {
          acc = 0;
          acc_phase ^= 1u;
        }
        continue;
      }
#endif
      for (int c0 = 0; c0 < p.CO; c0 += kColsPerStep) {
        uint32_t v[32];
        uint32_t packed[32];
        tmem_ld_32x32(t_addr + c0, v);
        tmem_ld_wait();
        if (OUT_BYTES == 4) {
#pragma unroll
          for (int i = 0; i < 32; ++i) packed[i] = v[i];
        } else {
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            __half2 h = __floats2half2_rn(__uint_as_float(v[2 * i]), __uint_as_float(v[2 * i + 1]));
            packed[i] = *reinterpret_cast<uint32_t*>(&h);
          }
          tmem_ld_32x32(t_addr + c0 + 32, v);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            __half2 h = __floats2half2_rn(__uint_as_float(v[2 * i]), __uint_as_float(v[2 * i + 1]));
            packed[16 + i] = *reinterpret_cast<uint32_t*>(&h);
          }
        }
        if (c0 + kColsPerStep >= p.CO) {
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(smem_u32(&bars->tmem_empty[acc]));
        }
        if (valid && p.out_nchw) {
          // channel-major output: consecutive lanes are consecutive pixels of one image row
          const long long plane = static_cast<long long>(p.HO) * p.WO;
          uint8_t* o = static_cast<uint8_t*>(p.out) +
                       ((static_cast<long long>(n) * p.CO + c0) * plane + static_cast<long long>(y) * p.WO + px) * OUT_BYTES;
#pragma unroll
          for (int i = 0; i < kColsPerStep; ++i) {
            if (OUT_BYTES == 4)
              *reinterpret_cast<uint32_t*>(o + i * plane * OUT_BYTES) = packed[i % 32];
            else
              *reinterpret_cast<uint16_t*>(o + i * plane * OUT_BYTES) =
                  static_cast<uint16_t>(packed[(i >> 1) % 32] >> (16 * (i & 1)));
          }
        } else if (valid) {
#pragma unroll
          for (int j = 0; j < 8; ++j)
            *reinterpret_cast<uint4*>(orow + c0 * OUT_BYTES + 16 * j) =
                make_uint4(packed[4 * j], packed[4 * j + 1], packed[4 * j + 2], packed[4 * j + 3]);
        }
      }
      if (++acc == 2) {
        acc = 0;
        acc_phase ^= 1u;
      }
    }
    __syncwarp();
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_cg<1>(tmem_base, static_cast<uint32_t>(p.tmem_cols));
  }
  if (threadIdx.x == 0 && *abort_flag) atomicExch(&g_hb_status, kErrTimeout);
}

}  // namespace hb
