// Stride-1 NHWC conv2d, resident filter, with the output CHANNELS on the MMA's M axis and up to 256
// output PIXELS on its N axis ("wide strip" algorithm, conv_algo 3).
//
// The strip kernel of hb_conv_strip.cuh puts 128 pixels on M and the CO output channels on N.  With
// CO = 64 every tcgen05.mma then carries a quarter of the work of a 128 x 256 one and costs about
// the same, so the tensor pipe idles three quarters of the time.  Here the operands change
// places:
//   A (M side) = one (tap, 64-channel chunk) slab of the HWIO filter, resident in shared memory:
//                K = input channels, M = output channels contiguous (an "MN-major" A operand);
//   B (N side) = the padded input strip: N = consecutive pixels, K = channels contiguous.
// Output positions are numbered in padded-linear order i = y * Wp + x (x < Wp = W + 2 * pad_w), as in
// the strip kernel, so filter tap (ry, rx) is the same strip read (ry*dil*Wp + rx*dil) pixels
// further on and B's descriptor just starts there.  Because the order is linear, a tile need not
// be made of whole image rows: a tile is any L = 256 consecutive positions of one image (the last
// tile of an image is shorter), which fills the MMA's N axis whatever the image width.
//
// The accumulator is D[channel][position]: with M = 64 the hardware keeps channel c in TMEM lane
// 32 * (c / 16) + c % 16 (16 lanes of each 32-lane quarter), with M = 128 in lane c.  An epilogue
// thread therefore owns one channel and reads 32 consecutive positions per tcgen05.ld, while the
// NHWC output wants, per position, all channels side by side.  The four epilogue warps transpose
// through shared memory: each writes its channels of the tile into a staging buffer laid out
// [position][channel] and arrives on a barrier; one thread waits for all eight and sends the tile
// out with bulk copies (cp.async.bulk shared -> global): the real pixels of an image row are
// contiguous both in the buffer and in the output, so a tile is one copy per image row it touches,
// and junk positions (x >= WO) are simply not part of any.  (Stores of 2 or 32 bytes scattered over
// many lines were measured at about one sector per 2 ns and SM: 60 us for this layer's 12.8 MB.)
// The copies read the buffer while the warps already fetch the next tile's accumulator; a second
// barrier tells them when the buffer may be overwritten.
//
// The filter arrives tap by tap, each tap on a barrier of its own, so that the first tile's MMAs
// start when the first 8 KiB slab is in, not the whole filter.
//
// Roles, barriers and the bounded-wait / abort protocol are those of hb_conv_strip.cuh.
#pragma once
#include "hb_conv_strip.cuh"

namespace hb {

constexpr int kMaxStripTRing = 4;
constexpr int kFiltBars = 16;      // filter taps with a barrier of their own (later taps share the last)
constexpr int kWideEpiWarps = 8;   // two per TMEM lane quarter: each takes half of a block's positions
constexpr int kWideThreads = 32 * (2 + kWideEpiWarps);

struct StripTParams {
  int N, H, W, CI, CO, KH, KW, pad_h, pad_w, dil_h, dil_w, HO, WO;
  int Wp;             // padded width
  int P;              // padded-linear output positions per image: (HO - 1) * Wp + WO
  int L;              // positions per tile (multiple of 16, <= 256)
  int tiles_per_img;  // ceil(P / L)
  int num_tiles;
  int SR;             // input rows per strip: enough for L positions from any column, plus the taps
  int strip_bytes;    // bytes per channel chunk of a strip (multiple of 1024)
  int n_cchunks;      // 128-byte channel chunks per pixel
  int esize_out;
  int tmem_cols;
  int ring;           // strip buffers in flight (2..kMaxStripTRing)
  long long wait_limit_cycles;
  int probe;          // diagnostic bits of -DHB_PROBES builds: 1 = no MMAs, 2 = no global stores, 4 = strips loaded
                      // once, 8 = no staging writes, 16 = no staging barrier, 32 = no copy-out loop
  uint32_t idesc;     // instruction descriptor without its N field
  void* out;
};

struct StripTBars {
  uint64_t filt_full[kFiltBars];
  uint64_t stage;       // the epilogue warps: "my channels of this tile are in the staging buffer"
  uint64_t stage_free;  // the copying thread: "the bulk copies have read the staging buffer"
  uint64_t strip_full[kMaxStripTRing];
  uint64_t strip_empty[kMaxStripTRing];
  uint64_t tmem_full[2];
  uint64_t tmem_empty[2];
  uint64_t drain;
  uint32_t tmem_base;
  int abort_flag;
};

template <int OUT_BYTES>
__global__ void __launch_bounds__(kWideThreads, 1)
hb_conv_strip_t_kernel(const __grid_constant__ CUtensorMap tmIn, const __grid_constant__ CUtensorMap tmW,
                       const StripTParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (smem_base - smem_u32(smem_raw));

  constexpr int BK = 64;                    // fp16 channels per 128-byte chunk
  const int tap_bytes = BK * p.CO * 2;      // one (tap, channel chunk) slab of the filter
  const int n_taps = p.KH * p.KW;
  const int filt_bytes = n_taps * p.n_cchunks * tap_bytes;
  const int strip_total = p.n_cchunks * p.strip_bytes;
  const uint32_t sFilt = smem_base;
  const uint32_t sStrip = sFilt + ((filt_bytes + 1023) & ~1023);
  const uint32_t sStage = sStrip + p.ring * strip_total;  // one tile: L pixels of CO * OUT_BYTES bytes
  const int stage_bytes = p.L * p.CO * OUT_BYTES;
  StripTBars* bars = reinterpret_cast<StripTBars*>(smem + (sStage - smem_base) + stage_bytes);
  volatile int* abort_flag = &bars->abort_flag;
  const WaitCtx wctx{abort_flag, p.wait_limit_cycles > 0 ? p.wait_limit_cycles : HB_WAIT_LIMIT_CYCLES};

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int i = 0; i < kFiltBars; ++i) mbar_init(smem_u32(&bars->filt_full[i]), 1);
    mbar_init(smem_u32(&bars->stage), kWideEpiWarps);
    mbar_init(smem_u32(&bars->stage_free), 1);
    for (int i = 0; i < kMaxStripTRing; ++i) {
      mbar_init(smem_u32(&bars->strip_full[i]), 1);
      mbar_init(smem_u32(&bars->strip_empty[i]), 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(smem_u32(&bars->tmem_full[i]), 1);
      mbar_init(smem_u32(&bars->tmem_empty[i]), kWideEpiWarps);
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
  griddep_wait();
  griddep_launch_dependents();

  // tile -> image, first position, number of positions
  auto tile_of = [&](int t, int& n, int& i0, int& len) {
    n = t / p.tiles_per_img;
    i0 = (t - n * p.tiles_per_img) * p.L;
    len = min(p.L, p.P - i0);
  };

  if (warp == 0) {
    // ------------------------------ producer ----------------------------------------------
    if (elect_one()) {
      bool ok = true;
      // the filter, once: per (tap, channel chunk) BK rows of K, each CO * 2 bytes of output
      // channels wide, fetched as CO * 2 / 128 boxes of 128 bytes
      const int n_mchunks = p.CO * 2 / 128;
      auto load_filter = [&]() {
      for (int tap = 0; tap < n_taps; ++tap) {
        const int fb = tap < kFiltBars ? tap : kFiltBars - 1;
        const uint32_t ff = smem_u32(&bars->filt_full[fb]);
        // (the last barrier takes every tap from kFiltBars - 1 on: armed once, with all their bytes)
        if (tap < kFiltBars)
          mbar_arrive_expect_tx(ff, static_cast<uint32_t>(p.n_cchunks * tap_bytes) *
                                        static_cast<uint32_t>(tap == kFiltBars - 1 ? n_taps - tap : 1));
        for (int cc = 0; cc < p.n_cchunks; ++cc)
          for (int j = 0; j < n_mchunks; ++j)
            tma_load_3d(sFilt + (tap * p.n_cchunks + cc) * tap_bytes + j * (BK * 128), &tmW, ff, j * 64,
                        tap * p.CI + cc * BK, 0);
      }
      // barriers of taps the filter does not have complete at once, so that every wait on them passes
      for (int fb = n_taps; fb < kFiltBars; ++fb) mbar_arrive(smem_u32(&bars->filt_full[fb]));
      };
      // (the first tile's strip goes out before the filter: TMA serves its requests in order, and
      // the first MMA needs the strip and one tap, not the whole filter)
      int buf = 0;
      uint32_t phase = 0;
      int issued = 0;
      const uint32_t tx = static_cast<uint32_t>(p.n_cchunks * p.SR * p.Wp * 128);
      for (int t = blockIdx.x; ok && t < p.num_tiles; t += gridDim.x) {
        int n, i0, len;
        tile_of(t, n, i0, len);
        const int y_first = i0 / p.Wp;
        if (!mbar_wait(smem_u32(&bars->strip_empty[buf]), phase ^ 1u, wctx)) {
          ok = false;
          break;
        }
        const uint32_t full = smem_u32(&bars->strip_full[buf]);
#ifdef HB_PROBES
        if ((p.probe & 4) && issued >= p.ring) {
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
                      y_first - p.pad_h, n);
        if (issued == 0) load_filter();
        ++issued;
        if (++buf == p.ring) {
          buf = 0;
          phase ^= 1u;
        }
      }
      if (issued == 0) load_filter();  // (a CTA without tiles: its barriers still complete)
      if (!ok) {
        for (int fb = 0; fb < kFiltBars; ++fb) mbar_wait_drain(smem_u32(&bars->filt_full[fb]), 0u);
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
      bool ok = true;
      bool filter_in = false;  // after the first tile every tap has been waited for
      int buf = 0, acc = 0;
      uint32_t phase = 0, acc_phase = 0;
      // A (filter): MN-major, 128-byte rows of output channels, 8-row K groups 1024 bytes apart,
      // 64-channel column chunks BK * 128 bytes apart; one MMA takes 16 K rows = 2048 bytes.
      // B (strip): K-major rows of 128 bytes, 8-row groups 1024 bytes apart; one MMA takes 32 bytes
      // of each row.
      const uint64_t desc_hi = static_cast<uint64_t>((1024u >> 4) | (1u << 14) | (2u << 29)) << 32;
      const uint32_t a_lo_fixed = ((static_cast<uint32_t>(BK * 128) >> 4) & 0x3FFFu) << 16;
      const uint32_t b_lo_fixed = (16u >> 4) << 16;
      const uint32_t a_step16 = (16u * 128u) >> 4;
      const uint32_t slab16 = static_cast<uint32_t>(tap_bytes) >> 4;                 // next (tap, chunk) slab of A
      const uint32_t chunk16 = static_cast<uint32_t>(p.strip_bytes) >> 4;            // next channel chunk of B
      const uint32_t tap_step16 = static_cast<uint32_t>(p.dil_w) * 8u;               // next tap of a filter row
      const uint32_t row_step16 = static_cast<uint32_t>(p.dil_h * p.Wp) * 8u;        // next filter row
      for (int t = blockIdx.x; ok && t < p.num_tiles; t += gridDim.x) {
        int n, i0, len;
        tile_of(t, n, i0, len);
        const int x0 = i0 - (i0 / p.Wp) * p.Wp;
        const uint32_t n_mma = static_cast<uint32_t>((len + 15) & ~15);
        const uint32_t idesc = p.idesc | ((n_mma >> 3) << 17);
        if (!mbar_wait(smem_u32(&bars->tmem_empty[acc]), acc_phase ^ 1u, wctx) ||
            !mbar_wait(smem_u32(&bars->strip_full[buf]), phase, wctx)) {
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc * 256);
        uint32_t accum = 0u;
        int kh = p.KH;
#ifdef HB_PROBES
        if (p.probe & 1) kh = 0;
        if (p.probe & 64) {
          // diagnostic: the tile's MMA count on fixed descriptors, no address arithmetic in the loop
          kh = 0;
          const uint32_t a_lo = ((sFilt >> 4) & 0x3FFFu) | a_lo_fixed;
          const uint32_t b_lo = (((sStrip + buf * strip_total) >> 4) & 0x3FFFu) | b_lo_fixed;
          const uint64_t da = desc_hi | a_lo, db = desc_hi | b_lo;
          const int nm = p.KH * p.KW * p.n_cchunks * 4;
          umma_cg<1, 0>(d_tmem, da, db, idesc, 0u);
#pragma unroll 4
          for (int i = 1; i < nm; ++i) umma_cg<1, 0>(d_tmem, da, db, idesc, 1u);
        }
#endif
        // Descriptor low words advance by running additions (16-byte units; shared memory is
        // < 256 KiB, so the 14-bit address field cannot wrap): per tap B moves on by dil_w pixels, per
        // filter row by dil_h padded rows, A by one (tap, chunk) slab.
        uint32_t a_lo = (sFilt >> 4) | a_lo_fixed;
        uint32_t b_row = (((sStrip + buf * strip_total) >> 4) + static_cast<uint32_t>(x0) * 8u) | b_lo_fixed;
        int tap = 0;
        for (int ry = 0; ry < kh && ok; ++ry, b_row += row_step16) {
          uint32_t b_tap = b_row;
          for (int rx = 0; rx < p.KW; ++rx, ++tap, b_tap += tap_step16) {
            if (!filter_in) {
              if (tap < kFiltBars && !mbar_wait(smem_u32(&bars->filt_full[tap]), 0u, wctx)) {
                ok = false;
                break;
              }
              tc_fence_after();
            }
            uint32_t b_lo = b_tap;
            for (int cc = 0; cc < p.n_cchunks; ++cc, a_lo += slab16, b_lo += chunk16) {
#pragma unroll
              for (int k = 0; k < 4; ++k) {
                umma_cg<1, 0>(d_tmem, desc_hi | (a_lo + a_step16 * k), desc_hi | (b_lo + 2u * k), idesc, accum);
                accum = 1u;
              }
            }
          }
        }
        if (!ok) break;
        filter_in = true;
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
    // Eight warps: warp w may read TMEM lane quarter w % 4; of the two warps of a quarter one takes
    // the first half of the tile's positions, the other the second half.
    const int q = warp & 3;
    const int half = (warp - 2) >> 2;
    const bool copier = threadIdx.x == 64;  // lane 0 of the first epilogue warp issues the bulk copies
    int acc = 0;
    uint32_t acc_phase = 0, stage_phase = 0, free_phase = 0;
    bool ok = true;
    bool copies_pending = false;
    // the channel this thread's TMEM lane holds (see the layout note at the top)
    const bool narrow = p.CO == 64;
    const int ch = narrow ? q * 16 + lane : q * 32 + lane;
    const bool lane_valid = !narrow || lane < 16;
    const int px_bytes = p.CO * OUT_BYTES;
    const uint32_t stage_bar = smem_u32(&bars->stage), free_bar = smem_u32(&bars->stage_free);
    const int half_len = ((p.L / 2 + 31) / 32) * 32;  // positions of the first warp half: whole 32-position chunks
    for (int t = blockIdx.x; ok && t < p.num_tiles; t += gridDim.x) {
      int n, i0, len;
      tile_of(t, n, i0, len);
      if (copier && copies_pending) {
        // the previous tile's copies have read the staging buffer: it may be overwritten
        bulk_wait_read<0>();
        mbar_arrive(free_bar);
        copies_pending = false;
      }
      if (!mbar_wait_relaxed(smem_u32(&bars->tmem_full[acc]), acc_phase, wctx)) {
        ok = false;
        break;
      }
      tc_fence_after();
      const int p0 = half * half_len;              // this warp's first position of the tile
      const int my_len = min(half_len, len - p0);  // (<= 0: none)
      const uint32_t t_addr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) +
                              static_cast<uint32_t>(acc * 256 + p0);
      uint8_t* img = static_cast<uint8_t*>(p.out) + static_cast<long long>(n) * p.HO * p.WO * px_bytes;
      // software pipeline over 32-position chunks: the TMEM load of chunk k + 1 is in flight while
      // chunk k goes to the staging buffer
      uint32_t v[32];
      if (my_len > 0) tmem_ld_32x32(t_addr, v);
      // (free_phase counts tiles: the buffer starts out free, so the first wait passes at once)
      if (!mbar_wait(free_bar, free_phase ^ 1u, wctx)) {
        tmem_ld_wait();  // (no TMEM load stays in flight past the loop)
        ok = false;
        break;
      }
      free_phase ^= 1u;
      for (int c = 0; c < my_len; c += 32) {
        uint32_t cur[32];
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 32; ++j) cur[j] = v[j];
        if (c + 32 < my_len) tmem_ld_32x32(t_addr + c + 32, v);
#ifdef HB_PROBES
        const bool store_ok = lane_valid && !(p.probe & 8);
#else
        const bool store_ok = lane_valid;
#endif
        if (OUT_BYTES == 4) {
          if (store_ok) {
            const uint32_t dst = sStage + static_cast<uint32_t>((p0 + c) * px_bytes + ch * 4);
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              if (c + j >= my_len) break;  // (the tile's last chunk may be short)
              asm volatile("st.shared.b32 [%0], %1;" ::"r"(dst + j * px_bytes), "r"(cur[j]) : "memory");
            }
          }
        } else {
          // fp16: two channels make one 32-bit word.  Lanes 2k and 2k + 1 hold channels c and c + 1;
          // they swap half of their values, after which the even lane holds both channels of the
          // chunk's even positions and the odd lane those of the odd positions: half as many stores,
          // none of them narrower than a bank word.
          const int odd = lane & 1;
          const uint32_t dst = sStage + static_cast<uint32_t>((p0 + c + odd) * px_bytes + (ch & ~1) * 2);
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const uint32_t keep = odd ? cur[2 * j + 1] : cur[2 * j];
            const uint32_t give = odd ? cur[2 * j] : cur[2 * j + 1];
            const uint32_t got = __shfl_xor_sync(0xffffffffu, give, 1);
            const __half2 h = odd ? __floats2half2_rn(__uint_as_float(got), __uint_as_float(keep))
                                  : __floats2half2_rn(__uint_as_float(keep), __uint_as_float(got));
            if (store_ok && c + 2 * j + odd < my_len)
              asm volatile("st.shared.b32 [%0], %1;" ::"r"(dst + 2 * j * px_bytes),
                           "r"(*reinterpret_cast<const uint32_t*>(&h))
                           : "memory");
          }
        }
      }
      // this accumulator has been read: hand it back to the MMA warp
      tc_fence_before();
      fence_proxy_async_smem();  // the staging writes above are read by bulk copies (async proxy)
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(smem_u32(&bars->tmem_empty[acc]));
        mbar_arrive(stage_bar);
      }
      if (copier) {
        // ---- every warp's channels of this tile are staged: whole pixels out, one bulk copy per
        //      image row the tile touches ----
        if (!mbar_wait(stage_bar, stage_phase, wctx)) {
          ok = false;
        } else {
          int i = i0;
          int y = i / p.Wp;
          int x = i - y * p.Wp;
          int done = 0;
          while (done < len) {
            const int in_row = min(len - done, p.Wp - x);  // positions of this tile left in row y
            const int valid = min(in_row, p.WO - x);        // ... of which real pixels (may be <= 0)
#ifdef HB_PROBES
            if (valid > 0 && !(p.probe & 2))
#else
            if (valid > 0)
#endif
              bulk_store(img + (static_cast<long long>(y) * p.WO + x) * px_bytes,
                         sStage + static_cast<uint32_t>(done * px_bytes), static_cast<uint32_t>(valid * px_bytes));
            done += in_row;
            x = 0;
            ++y;
          }
          bulk_commit();
          copies_pending = true;
        }
      }
      stage_phase ^= 1u;
      ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;  // (the copier's result counts for its warp)
      if (++acc == 2) {
        acc = 0;
        acc_phase ^= 1u;
      }
    }
    if (copier) bulk_wait_read<0>();  // shared memory must outlive the copies' reads of it
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
