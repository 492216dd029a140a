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
// Roles as in hb_umma_kernel: warp 0 loads (the first strip, then the filter tap by tap, each tap
// on a barrier of its own, then strips into a ring of two to six buffers), warp 1 issues MMAs into
// one of two TMEM accumulators (descriptor words advance by running additions), warps 2..5 read
// the accumulator.  An M = 128, N = 64, K = 16 MMA on fresh operands takes about 50 ns here, which is
// its 6 KB of operands at the ~64 bytes per cycle the tensor core draws from shared memory, not
// the issue loop: the same MMA repeated on the same descriptors takes 30 ns.
// Each epilogue thread owns one output pixel (CO contiguous elements).  Staged epilogue (NHWC
// output whose tile fits shared memory): the thread writes its pixel, 128 bytes of channels at a
// time, into a 128-byte-swizzled staging buffer laid out [row][x][channels] with the junk positions
// squeezed out (conflict-free 16-byte stores), the four warps meet at a barrier and one thread
// sends the tile out with one tiled TMA store per 128-byte channel chunk: box (channels, WO, R),
// rows past the image clipped by TMA.  Direct epilogue (channel-major output, or no room): the
// thread stores its pixel itself, which touches 32 lines per warp instruction and runs at about
// one sector per 2 ns and SM.  All waits are bounded, with the same abort protocol.
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
              // back, 4 = strips loaded once, 9 = the tile's MMAs on fixed descriptors (and 3); fused form
              // only: 5 = no boundary exchange, 6 = no shifted adds, 7 = no staging writes and no TMA stores
  uint32_t idesc;
  void* out;
  int out_nchw;  // output is (N, CO, HO, WO) instead of (N, HO, WO, CO)
  int staged;    // 1: the epilogue goes through the staging buffer and TMA stores (see above)
  int stage_chunk_bytes;  // staging bytes per 128-byte channel chunk: R * WO * 128, rounded up to 1024
  int fuse_kw;   // 1: the KW taps of a filter row share one MMA of N = KW * CO columns (see FUSE below)
  int acc_cols;  // TMEM columns from one accumulator to the other: CO, or KW * CO when fused
};

// Shared memory of the fused form's boundary exchange: per warp group and tile parity, per 32
// TMEM lanes, the second and third column groups of their first position and the third of
// their second (two parities: a fast warp publishes for the group's next tile while a slow one
// still reads this tile's rows).
constexpr int kStripXchRows = 3;
constexpr int kStripFusedEpiWarps = 8;  // two groups of four: one drains a tile while the other drains the next
constexpr int kStripFusedThreads = 32 * (2 + kStripFusedEpiWarps);
__host__ __device__ constexpr int strip_xch_bytes(int co) { return 2 * 2 * 4 * kStripXchRows * co * 4; }


constexpr int kStripFiltBars = 16;  // filter taps with a barrier of their own (later taps share the last)

struct StripBars {
  uint64_t filt_full[kStripFiltBars];
  // (one of each per epilogue warp group: the fused form has two groups that take tiles in turn)
  uint64_t stage[2];       // the epilogue warps: "my pixels of this tile are in the staging buffer"
  uint64_t stage_free[2];  // the copying thread: "the TMA stores have read the staging buffer"
  uint64_t xch[2];         // fused form: "my first positions' column groups of this tile are published"
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

// Tiled 4-D store from shared memory (bulk-group completion); elements past the tensor are dropped.
__device__ __forceinline__ void tma_store_4d(const CUtensorMap* m, uint32_t src, int c, int w, int h, int n) {
  asm volatile(
      "cp.async.bulk.tensor.4d.global.shared::cta.bulk_group [%0, {%2, %3, %4, %5}], [%1];" ::"l"(
          reinterpret_cast<uint64_t>(m)),
      "r"(src), "r"(c), "r"(w), "r"(h), "r"(n)
      : "memory");
}

// FUSE = 1 (fp16, one 128-byte chunk of output channels, KW = 3, dilation 1 along W): the three
// taps of a filter row are consecutive slabs of the resident filter, so one MN-major descriptor
// with the slab distance as its column-chunk stride reads them as one B operand of 3 * CO
// columns.  The MMA of filter row ry then takes the strip at the row's first tap as A and leaves,
// in column group g, tap (ry, g) applied to the pixel g places to the LEFT of where it belongs:
//   out[pos] = G0[pos] + G1[pos + 1] + G2[pos + 2].
// A tile is whole padded rows and an output row ends KW - 1 pixels before its padded row, so the
// shifted reads never leave the tile.  A third of the MMAs, each fetching 10 KB of operands for
// 128 x 192 x 16 products instead of 6 KB for 128 x 64 x 16.  Positions are TMEM lanes: the
// epilogue shifts with warp shuffles, and a warp's last two lanes take the next warp's first two
// positions from a small shared-memory exchange (double-buffered by tile parity, published
// behind an mbarrier so that the wait is bounded like every other).  Eight epilogue warps in two
// groups of four: group g drains the CTA's tiles g, g + 2, ... from accumulator g through its own
// staging tile, barriers and copying thread, so that one tile's drain overlaps the next one's.
template <int OUT_BYTES, int KIND, int FUSE = 0>
__global__ void __launch_bounds__(FUSE ? kStripFusedThreads : kThreads, 1)
hb_conv_strip_kernel(const __grid_constant__ CUtensorMap tmIn, const __grid_constant__ CUtensorMap tmW,
                     const __grid_constant__ CUtensorMap tmOut, const StripParams p) {
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
  const uint32_t sStage = sStrip + p.ring * strip_total;  // 1024-byte aligned: strips are multiples of 1024
  const int n_ochunks = p.CO * OUT_BYTES / 128;           // 128-byte channel chunks of an output pixel
  const int stage_bytes = p.staged ? n_ochunks * p.stage_chunk_bytes : 0;
  // (the fused form has a staging buffer per epilogue warp group)
  StripBars* bars = reinterpret_cast<StripBars*>(smem + (sStage - smem_base) + (FUSE ? 2 : 1) * stage_bytes);
  float* const xch_base = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(bars) + 512);  // fused form only
  volatile int* abort_flag = &bars->abort_flag;
  const WaitCtx wctx{abort_flag, p.wait_limit_cycles > 0 ? p.wait_limit_cycles : HB_WAIT_LIMIT_CYCLES};

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int i = 0; i < kStripFiltBars; ++i) mbar_init(smem_u32(&bars->filt_full[i]), 1);
    for (int g = 0; g < 2; ++g) {
      mbar_init(smem_u32(&bars->stage[g]), kEpiWarps);
      mbar_init(smem_u32(&bars->stage_free[g]), 1);
      mbar_init(smem_u32(&bars->xch[g]), kEpiWarps);
    }
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
    if (p.staged) prefetch_tmap(&tmOut);
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
      auto load_filter = [&]() {
        for (int tap = 0; tap < n_taps; ++tap) {
          const int fb = tap < kStripFiltBars ? tap : kStripFiltBars - 1;
          const uint32_t ff = smem_u32(&bars->filt_full[fb]);
          // (the last barrier takes every tap from kStripFiltBars - 1 on: armed once, with all their bytes)
          if (tap < kStripFiltBars)
            mbar_arrive_expect_tx(ff, static_cast<uint32_t>(p.n_cchunks * tap_bytes) *
                                          static_cast<uint32_t>(tap == kStripFiltBars - 1 ? n_taps - tap : 1));
          for (int cc = 0; cc < p.n_cchunks; ++cc)
            for (int j = 0; j < n_nchunks; ++j)
              tma_load_3d(sFilt + (tap * p.n_cchunks + cc) * tap_bytes + j * (BK * 128), &tmW, ff,
                          j * chunk_cols, tap * p.CI + cc * BK, 0);
        }
        // barriers of taps the filter does not have complete at once, so that every wait on them passes
        for (int fb = n_taps; fb < kStripFiltBars; ++fb) mbar_arrive(smem_u32(&bars->filt_full[fb]));
      };
      // (the first tile's strip goes out before the filter: TMA serves its requests in order, and the
      // first MMA needs the strip and one tap, not the whole filter)
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
        if (issued == 0) load_filter();
        ++issued;
        if (++buf == p.ring) {
          buf = 0;
          phase ^= 1u;
        }
      }
      if (issued == 0) load_filter();  // (a CTA without tiles: its barriers still complete)
      if (!ok) {
        for (int fb = 0; fb < kStripFiltBars; ++fb) mbar_wait_drain(smem_u32(&bars->filt_full[fb]), 0u);
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
      const int umma_k = 32 / p.esize_in;
      // A: K-major rows of 128 bytes, 8-row groups 1024 bytes apart.  B: MN-major, 128-byte
      // rows of output channels, 8-row groups 1024 bytes apart, column chunks BK*128 bytes apart.
      const uint64_t desc_hi = static_cast<uint64_t>((1024u >> 4) | (1u << 14) | (2u << 29)) << 32;
      const uint32_t a_lo_fixed = (16u >> 4) << 16;
      const uint32_t b_lo_fixed = ((static_cast<uint32_t>(BK * 128) >> 4) & 0x3FFFu) << 16;
      const uint32_t b_step16 = static_cast<uint32_t>(umma_k * 128) >> 4;
      const uint32_t idesc = p.idesc;
      // running steps of the descriptor low words, in 16-byte units (shared memory is < 256 KiB, so
      // the 14-bit address field cannot wrap)
      const uint32_t slab16 = static_cast<uint32_t>(tap_bytes) >> 4;            // next (tap, chunk) slab of B
      const uint32_t chunk16 = static_cast<uint32_t>(p.strip_bytes) >> 4;       // next channel chunk of A
      const uint32_t tap_step16 = static_cast<uint32_t>(p.dil_w) * 8u;          // next tap of a filter row
      const uint32_t row_step16 = static_cast<uint32_t>(p.dil_h * p.Wp) * 8u;   // next filter row
      for (int t = blockIdx.x; ok && t < p.num_tiles; t += gridDim.x) {
        if (!mbar_wait(smem_u32(&bars->tmem_empty[acc]), acc_phase ^ 1u, wctx) ||
            !mbar_wait(smem_u32(&bars->strip_full[buf]), phase, wctx)) {
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc * p.acc_cols);
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
        if constexpr (FUSE) {
          // one MMA per (filter row, channel chunk, 32 bytes of K): B's column chunks are the row's
          // taps, n_cchunks slabs apart
          const uint32_t b_fused = ((static_cast<uint32_t>(p.n_cchunks * tap_bytes) >> 4) & 0x3FFFu) << 16;
          uint32_t b_row = (sFilt >> 4) | b_fused;
          uint32_t a_row = ((sStrip + buf * strip_total) >> 4) | a_lo_fixed;
          const uint32_t b_row_step16 = static_cast<uint32_t>(p.KW * p.n_cchunks) * slab16;
          for (int ry = 0; ry < p.KH && ok; ++ry, a_row += row_step16, b_row += b_row_step16) {
            if (!filter_in) {
              for (int rx = 0; rx < p.KW && ok; ++rx) {
                const int tap = ry * p.KW + rx;
                if (tap < kStripFiltBars && !mbar_wait(smem_u32(&bars->filt_full[tap]), 0u, wctx)) ok = false;
              }
              if (!ok) break;
              tc_fence_after();
            }
            uint32_t a_lo = a_row, b_lo = b_row;
            for (int cc = 0; cc < p.n_cchunks; ++cc, a_lo += chunk16, b_lo += slab16) {
#pragma unroll
              for (int k = 0; k < 4; ++k) {
                umma_cg<1, KIND>(d_tmem, desc_hi | (a_lo + 2u * k), desc_hi | (b_lo + b_step16 * k), idesc, accum);
                accum = 1u;
              }
            }
          }
        } else {
          uint32_t b_lo = (sFilt >> 4) | b_lo_fixed;
          uint32_t a_row = ((sStrip + buf * strip_total) >> 4) | a_lo_fixed;
          int tap = 0;
          for (int ry = 0; ry < p.KH && ok; ++ry, a_row += row_step16) {
            uint32_t a_tap = a_row;
            for (int rx = 0; rx < p.KW; ++rx, ++tap, a_tap += tap_step16) {
              if (!filter_in) {
                if (tap < kStripFiltBars && !mbar_wait(smem_u32(&bars->filt_full[tap]), 0u, wctx)) {
                  ok = false;
                  break;
                }
                tc_fence_after();
              }
              uint32_t a_lo = a_tap;
              for (int cc = 0; cc < p.n_cchunks; ++cc, a_lo += chunk16, b_lo += slab16) {
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                  umma_cg<1, KIND>(d_tmem, desc_hi | (a_lo + 2u * k), desc_hi | (b_lo + b_step16 * k), idesc, accum);
                  accum = 1u;
                }
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
    const int q = warp & 3;
    // Fused form: two groups of four warps; group g drains the CTA's tiles g, g + 2, ... from
    // accumulator g into its own staging buffer, so one tile's drain overlaps the next one's.
    const int grp = FUSE ? (warp - 2) >> 2 : 0;
    int acc = grp;
    uint32_t acc_phase = 0, stage_phase = 0, free_phase = 0, xch_phase = 0;
    bool ok = true;
    bool copies_pending = false;
    const bool copier = threadIdx.x == 64 + 128 * grp;  // lane 0 of the group's first warp issues the TMA stores
    const uint32_t sStageG = sStage + static_cast<uint32_t>(grp * stage_bytes);
    constexpr int kColsPerStep = 128 / OUT_BYTES;  // 32 or 64 output channels = 128 bytes
    const int pos = q * 32 + lane;                 // padded-linear position inside the tile
    const int py = pos / p.Wp;
    const int px = pos - py * p.Wp;
    const int r2 = py * p.WO + px;                 // the pixel's row in the squeezed [R][WO] staging tile
    const uint32_t stage_bar = smem_u32(&bars->stage[grp]), free_bar = smem_u32(&bars->stage_free[grp]);
    const uint32_t xch_bar = smem_u32(&bars->xch[grp]);
    auto next_acc = [&]() {
      if (FUSE) {
        acc_phase ^= 1u;  // (a group keeps its accumulator)
      } else if (++acc == 2) {
        acc = 0;
        acc_phase ^= 1u;
      }
    };
    int it = 0;
    for (int t = blockIdx.x; ok && t < p.num_tiles; t += gridDim.x, ++it) {
      if (FUSE && (it & 1) != grp) continue;
      const int n = t / p.groups;
      const int y0 = (t - n * p.groups) * p.R;
      const int y = y0 + py;
      const bool valid = py < p.R && y < p.HO && px < p.WO;
      if (!FUSE && copier && copies_pending) {
        // the previous tile's stores have read the staging buffer: it may be overwritten
        bulk_wait_read<0>();
        mbar_arrive(free_bar);
        copies_pending = false;
      }
      if (!mbar_wait(smem_u32(&bars->tmem_full[acc]), acc_phase, wctx)) {
        ok = false;
        break;
      }
      tc_fence_after();
      const uint32_t t_addr =
          tmem_base + (static_cast<uint32_t>(q * 32) << 16) + static_cast<uint32_t>(acc * p.acc_cols);
      // fused form: this tile's exchange rows of this warp and of the next one (the last warp's
      // last two lanes are never output pixels; they read the first warp's rows and drop the sum)
      float* const xch_mine = xch_base + (((grp * 2 + xch_phase) * 4 + q) * kStripXchRows) * p.CO;
      const float* const xch_next = xch_base + (((grp * 2 + xch_phase) * 4 + ((q + 1) & 3)) * kStripXchRows) * p.CO;
      uint8_t* orow = static_cast<uint8_t*>(p.out) +
                      ((static_cast<long long>(n) * p.HO + y) * p.WO + px) * p.CO * OUT_BYTES;
#ifdef HB_PROBES
      if (p.probe == 3 || p.probe == 9) {
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&bars->tmem_empty[acc]));
        next_acc();
        continue;
      }
#endif
      if (!FUSE && p.staged) {
        // (free_phase counts tiles: the buffer starts out free, so the first wait passes at once)
        if (!mbar_wait(free_bar, free_phase ^ 1u, wctx)) {
          ok = false;
          break;
        }
        free_phase ^= 1u;
      }
      if constexpr (FUSE) {
        // out[pos] = G0[pos] + G1[pos + 1] + G2[pos + 2].  Shuffles inside the warp; its last two
        // lanes need the next warp's first two positions: every warp first puts the second and
        // third column groups of its own first two positions into the exchange rows of its 32
        // lanes, the group meets at a barrier, and every lane reads the next warp's rows (one or
        // two addresses per instruction: broadcasts) and selects without a branch: a divergent
        // branch per channel costs more than the rest of the drain.  (Publishing from the registers
        // of the main pass instead measured slower on the 56 x 56 x 64 layer: by 1.7 us with a
        // barrier per half, and by 2.1 us with one barrier after the main pass and the two boundary
        // lanes finishing their pixels from parked partial sums afterwards.)
        uint32_t g0[32], g1[32], g2[32];
#ifdef HB_PROBES
        // diagnostics (wrong results): 5 = no boundary exchange, 6 = no shifted adds, 7 = no staging
        // writes and no TMA stores
        if (p.probe != 5)
#endif
#pragma unroll
        for (int cb = 0; cb < 64; cb += 32) {
          tmem_ld_32x32(t_addr + p.CO + cb, g1);
          tmem_ld_32x32(t_addr + 2 * p.CO + cb, g2);
          tmem_ld_wait();
          // (rows of the exchange are CO * 4 = 256 bytes and start 256-byte aligned: vector stores)
          if (lane == 0) {
            uint4* dst = reinterpret_cast<uint4*>(xch_mine + cb);
#pragma unroll
            for (int i = 0; i < 8; ++i) dst[i] = make_uint4(g1[4 * i], g1[4 * i + 1], g1[4 * i + 2], g1[4 * i + 3]);
          }
          if (lane < 2) {
            uint4* dst = reinterpret_cast<uint4*>(xch_mine + (1 + lane) * p.CO + cb);
#pragma unroll
            for (int i = 0; i < 8; ++i) dst[i] = make_uint4(g2[4 * i], g2[4 * i + 1], g2[4 * i + 2], g2[4 * i + 3]);
          }
        }
        __syncwarp();
#ifdef HB_PROBES
        if (p.probe != 5)
#endif
        if (lane == 0) mbar_arrive(xch_bar);
        // (the first half's columns are in flight while the other warps publish)
        tmem_ld_32x32(t_addr, g0);
        tmem_ld_32x32(t_addr + p.CO, g1);
        tmem_ld_32x32(t_addr + 2 * p.CO, g2);
        if (copier && copies_pending) {
          // the stores of this group's previous tile have read its staging buffer (the wait sits
          // here, behind the exchange, so that it costs the group nothing when the stores are done)
          bulk_wait_read<0>();
          mbar_arrive(free_bar);
          copies_pending = false;
        }
#ifdef HB_PROBES
        if ((p.probe != 5 && !mbar_wait(xch_bar, xch_phase, wctx)) ||
#else
        if (!mbar_wait(xch_bar, xch_phase, wctx) ||
#endif
            (p.staged && !mbar_wait(free_bar, free_phase ^ 1u, wctx))) {
          tmem_ld_wait();
          ok = false;
          break;
        }
        if (p.staged) free_phase ^= 1u;
        const bool last = lane == 31, last2 = lane >= 30;
#pragma unroll
        for (int cb = 0; cb < 64; cb += 32) {
          const float4* r1 = reinterpret_cast<const float4*>(xch_next + cb);
          const float4* r2v = reinterpret_cast<const float4*>(xch_next + (1 + (lane & 1)) * p.CO + cb);
          uint32_t packed[32 * OUT_BYTES / 4];  // this position's 32 channels: 64 or 128 bytes
          tmem_ld_wait();
          if (cb == 32) {
            // Last read of this accumulator: hand it back to the MMA warp at once.
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&bars->tmem_empty[acc]));
          }
#pragma unroll
          for (int i4 = 0; i4 < 8; ++i4) {
            const float4 u = r1[i4], w = r2v[i4];
            const float n1[4] = {u.x, u.y, u.z, u.w}, n2[4] = {w.x, w.y, w.z, w.w};
            float sum[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) {
              const int i = 4 * i4 + k;
#ifdef HB_PROBES
              if (p.probe == 6) {
                sum[k] = __uint_as_float(g0[i]) + __uint_as_float(g1[i]) + __uint_as_float(g2[i]) + n1[k] + n2[k];
                continue;
              }
#endif
              const float a1 = __shfl_down_sync(0xffffffffu, __uint_as_float(g1[i]), 1);
              const float a2 = __shfl_down_sync(0xffffffffu, __uint_as_float(g2[i]), 2);
              sum[k] = (__uint_as_float(g0[i]) + (last ? n1[k] : a1)) + (last2 ? n2[k] : a2);
            }
            if (OUT_BYTES == 4) {
#pragma unroll
              for (int k = 0; k < 4; ++k) packed[(4 * i4 + k) % (32 * OUT_BYTES / 4)] = __float_as_uint(sum[k]);
            } else {
              __half2 h0 = __floats2half2_rn(sum[0], sum[1]), h1 = __floats2half2_rn(sum[2], sum[3]);
              packed[(2 * i4) % (32 * OUT_BYTES / 4)] = *reinterpret_cast<uint32_t*>(&h0);
              packed[(2 * i4 + 1) % (32 * OUT_BYTES / 4)] = *reinterpret_cast<uint32_t*>(&h1);
            }
          }
          if (cb == 0) {
            // (the second half's columns load while the first half is stored)
            tmem_ld_32x32(t_addr + 32, g0);
            tmem_ld_32x32(t_addr + p.CO + 32, g1);
            tmem_ld_32x32(t_addr + 2 * p.CO + 32, g2);
          }
          constexpr int kVecs = 32 * OUT_BYTES / 16;  // 16-byte pieces of these 32 channels: 4 or 8
          const int byte0 = cb * OUT_BYTES;           // where they start in the pixel's output
#ifdef HB_PROBES
          if (p.probe == 7) continue;
#endif
          if (p.staged) {
            if (valid) {
              const uint32_t row_addr =
                  sStageG + static_cast<uint32_t>((byte0 >> 7) * p.stage_chunk_bytes + r2 * 128);
              const int j0 = (byte0 & 127) >> 4;
#pragma unroll
              for (int j = 0; j < kVecs; ++j) {
                const uint32_t a = row_addr + (((j0 + j) ^ (r2 & 7)) << 4);
                asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(a), "r"(packed[4 * j]),
                             "r"(packed[4 * j + 1]), "r"(packed[4 * j + 2]), "r"(packed[4 * j + 3])
                             : "memory");
              }
            }
          } else if (valid && p.out_nchw) {
            const long long plane = static_cast<long long>(p.HO) * p.WO;
            uint8_t* o = static_cast<uint8_t*>(p.out) +
                         ((static_cast<long long>(n) * p.CO + cb) * plane + static_cast<long long>(y) * p.WO + px) * OUT_BYTES;
#pragma unroll
            for (int i = 0; i < 32; ++i) {
              if (OUT_BYTES == 4)
                *reinterpret_cast<uint32_t*>(o + i * plane * OUT_BYTES) = packed[i % (32 * OUT_BYTES / 4)];
              else
                *reinterpret_cast<uint16_t*>(o + i * plane * OUT_BYTES) =
                    static_cast<uint16_t>(packed[(i >> 1) % (32 * OUT_BYTES / 4)] >> (16 * (i & 1)));
            }
          } else if (valid) {
#pragma unroll
            for (int j = 0; j < kVecs; ++j)
              *reinterpret_cast<uint4*>(orow + byte0 + 16 * j) =
                  make_uint4(packed[4 * j], packed[4 * j + 1], packed[4 * j + 2], packed[4 * j + 3]);
          }
        }
      }
      for (int c0 = 0; !FUSE && c0 < p.CO; c0 += kColsPerStep) {
        uint32_t v[32];
        uint32_t packed[32];
        if (OUT_BYTES == 4) {
          tmem_ld_32x32(t_addr + c0, v);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) packed[i] = v[i];
        } else {
          tmem_ld_32x32(t_addr + c0, v);
          tmem_ld_wait();
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
        if (p.staged) {
          // this pixel's 128 bytes of channels, into row r2 of the chunk's swizzled staging tile
          if (valid) {
            const uint32_t row_addr =
                sStage + static_cast<uint32_t>((c0 / kColsPerStep) * p.stage_chunk_bytes + r2 * 128);
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              const uint32_t a = row_addr + ((j ^ (r2 & 7)) << 4);
              asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(a), "r"(packed[4 * j]),
                           "r"(packed[4 * j + 1]), "r"(packed[4 * j + 2]), "r"(packed[4 * j + 3])
                           : "memory");
            }
          }
        } else if (valid && p.out_nchw) {
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
      if (p.staged) {
        fence_proxy_async_smem();  // the staging writes above are read by TMA stores (async proxy)
        __syncwarp();
        if (lane == 0) mbar_arrive(stage_bar);
        if (copier) {
          // every warp's pixels of this tile are staged: one tiled store per 128-byte channel chunk,
          // box (channels, WO, R); rows past the image's last are clipped by TMA
          if (!mbar_wait(stage_bar, stage_phase, wctx)) {
            ok = false;
          } else {
#ifdef HB_PROBES
            if (p.probe != 7)
#endif
            for (int c = 0; c < n_ochunks; ++c)
              tma_store_4d(&tmOut, sStageG + static_cast<uint32_t>(c * p.stage_chunk_bytes), c * kColsPerStep, 0,
                           y0, n);
            bulk_commit();
            copies_pending = true;
          }
        }
        stage_phase ^= 1u;
        ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;  // (the copier's result counts for its warp)
      }
      if (FUSE) xch_phase ^= 1u;
      next_acc();
    }
    if (copier) bulk_wait_read<0>();  // shared memory must outlive the stores' reads of it
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
