// Plans for the convolutions: implicit GEMM over im2col TMA, the resident-filter strip kernel,
// the packed-filter (x86) form and the NCHW operators with their layout glue.
#pragma once
#include "hb_plan.cuh"
#include "hb_plan_strip_t.cuh"

namespace {

int conv_out_extent(int in, int k, int stride, int pad, int dil) {
  const int span = (k - 1) * dil + 1;
  return (in - span + 2 * pad) / stride + 1;
}



// Shared-memory need of the strip algorithm for a geometry, or 0 when it does not apply.  `fuse`:
// the form whose MMAs take the three taps of a filter row at once (fp16, 64 output channels,
// KW = 3, no dilation along W).
int strip_smem_bytes(const ConvGeom& g, int es, int eo, hb::StripParams* sp, bool fuse = false) {
  if (g.stride_h != 1 || g.stride_w != 1) return 0;
  if (fuse && (es != 2 || g.CO * es != 128 || g.KW != 3 || g.dil_w != 1)) return 0;
  if ((g.CI * es) % 128 != 0 || (g.CO * es) % 128 != 0) return 0;
  if (g.CO > 256 || g.CO % (128 / eo) != 0 || g.CO % 16 != 0) return 0;
  const int Wp = g.W + 2 * g.pad_w;
  if (Wp > 128 || Wp < 1) return 0;
  const int R = 128 / Wp;
  const int strip_rows = R + (g.KH - 1) * g.dil_h;
  if (strip_rows > 256) return 0;
  const int max_off = (g.KH - 1) * g.dil_h * Wp + (g.KW - 1) * g.dil_w;
  int px = strip_rows * Wp;
  if (max_off + 128 > px) px = max_off + 128;
  const int strip_bytes = (px * 128 + 1023) & ~1023;
  const int n_cchunks = g.CI * es / 128;
  const long long filt = static_cast<long long>(g.KH) * g.KW * g.CI * g.CO * es;
  long long smem = ((filt + 1023) & ~1023LL) + 2LL * n_cchunks * strip_bytes + 1024 + 512;
  if (fuse) smem += hb::strip_xch_bytes(g.CO);
  if (smem > kSmemLimit) return 0;
  // Staged epilogue (row-major output): one squeezed [R][WO] tile of 128-byte rows per 128-byte
  // channel chunk of the output, sent out by TMA.  It takes precedence over a deeper strip ring.
  const int stage_chunk = (R * g.WO * 128 + 1023) & ~1023;
  const long long stage = static_cast<long long>(g.CO) * eo / 128 * stage_chunk;
  // (the fused form drains two tiles at a time: a staging tile per epilogue warp group)
  const long long stage_all = (fuse ? 2 : 1) * stage;
  const bool staged = !g.out_nchw && g.WO <= 256 && R <= 256 && smem + stage_all <= kSmemLimit;
  if (staged) smem += stage_all;
  int ring = 2;  // deeper when shared memory allows: more strips in flight hide HBM latency
  while (ring < hb::kMaxStripRing && smem + static_cast<long long>(n_cchunks) * strip_bytes <= kSmemLimit) {
    smem += static_cast<long long>(n_cchunks) * strip_bytes;
    ++ring;
  }
  if (sp) {
    sp->ring = ring;
    sp->Wp = Wp; sp->R = R; sp->strip_rows = strip_rows; sp->strip_bytes = strip_bytes;
    sp->n_cchunks = n_cchunks; sp->groups = (g.HO + R - 1) / R;
    sp->staged = staged ? 1 : 0; sp->stage_chunk_bytes = stage_chunk;
    sp->fuse_kw = fuse ? 1 : 0; sp->acc_cols = fuse ? g.KW * g.CO : g.CO;
  }
  return static_cast<int>(smem);
}

int build_strip_plan(Driver& d, const ConvGeom& g, hb_dtype in_a, hb_dtype in_w, hb_dtype out_t,
                     const hb_knobs& k, const void* in, const void* w, void* out, hb_plan* plan) {
  const int es = esize(in_a), eo = esize(out_t);
  if (g_plan_owns_flags) release_split_flags(plan->p.flags, plan->owned_flags);
  std::memset(plan, 0, sizeof(*plan));
  hb::StripParams& sp = plan->sp;
  const bool fuse = k.conv_algo == 4;
  const int smem = strip_smem_bytes(g, es, eo, &sp, fuse);
  if (smem == 0 || (fuse && in_w != HB_F16)) return HB_ERR_KNOB;
  const long long tiles = static_cast<long long>(g.N) * sp.groups;
  if (tiles > 0x7fffffffLL) return HB_ERR_SHAPE;
  sp.N = g.N; sp.H = g.H; sp.W = g.W; sp.CI = g.CI; sp.CO = g.CO; sp.KH = g.KH; sp.KW = g.KW;
  sp.pad_h = g.pad_h; sp.pad_w = g.pad_w; sp.dil_h = g.dil_h; sp.dil_w = g.dil_w; sp.HO = g.HO; sp.WO = g.WO;
  sp.num_tiles = static_cast<int>(tiles);
  sp.esize_in = es; sp.esize_out = eo;
  sp.tmem_cols = next_pow2_cols(2 * sp.acc_cols);
  const int kind = mma_kind(in_a, in_w, out_t);
  sp.idesc = make_idesc(kind, in_a, in_w, hb::kTileM, sp.acc_cols, true);
  sp.out = out;
  sp.out_nchw = g.out_nchw ? 1 : 0;
  sp.probe = k.probe;
  // input as a tiled (C, W, H, N) tensor: one box = 128 bytes of channels x padded width x strip rows
  cuuint64_t dims[4] = {static_cast<cuuint64_t>(g.CI), static_cast<cuuint64_t>(g.W),
                        static_cast<cuuint64_t>(g.H), static_cast<cuuint64_t>(g.N)};
  cuuint64_t strides[3] = {static_cast<cuuint64_t>(g.CI) * es, static_cast<cuuint64_t>(g.W) * g.CI * es,
                           static_cast<cuuint64_t>(g.H) * g.W * g.CI * es};
  cuuint32_t box[4] = {static_cast<cuuint32_t>(128 / es), static_cast<cuuint32_t>(sp.Wp),
                       static_cast<cuuint32_t>(sp.strip_rows), 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = d.tiled(&plan->tmA, tmap_dtype(in_a), 4, const_cast<void*>(in), dims, strides, box, estr,
                       CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                       CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return HB_ERR_LAUNCH;
  const long long K = static_cast<long long>(g.KH) * g.KW * g.CI;
  const uint64_t rowB = static_cast<uint64_t>(g.CO) * es;
  int rc = encode_tiled3(d, &plan->tmB, in_w, w, g.CO, K, 1, rowB, rowB * K, 128 / es, 128 / es, 128);
  if (rc != HB_OK) return rc;
  plan->tmC = plan->tmA;  // (a valid map in every case; the staged epilogue gets the output's below)
  if (sp.staged) {
    // output as a tiled (C, W, H, N) tensor: one box = 128 bytes of channels x WO x R rows
    cuuint64_t odims[4] = {static_cast<cuuint64_t>(g.CO), static_cast<cuuint64_t>(g.WO),
                           static_cast<cuuint64_t>(g.HO), static_cast<cuuint64_t>(g.N)};
    cuuint64_t ostrides[3] = {static_cast<cuuint64_t>(g.CO) * eo, static_cast<cuuint64_t>(g.WO) * g.CO * eo,
                              static_cast<cuuint64_t>(g.HO) * g.WO * g.CO * eo};
    cuuint32_t obox[4] = {static_cast<cuuint32_t>(128 / eo), static_cast<cuuint32_t>(g.WO),
                          static_cast<cuuint32_t>(sp.R), 1};
    r = d.tiled(&plan->tmC, tmap_dtype(out_t), 4, out, odims, ostrides, obox, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return HB_ERR_LAUNCH;
  }
  int grid = d.sm_count;
  if (k.max_ctas > 0 && k.max_ctas < grid) grid = k.max_ctas;
  if (sp.num_tiles < grid) grid = sp.num_tiles;
  plan->strip = true;
  plan->grid = grid;
  plan->smem = smem;
  plan->knobs = k;
  plan->knobs.conv_algo = fuse ? 4 : 2;
  // fields hb_plan_knobs reports
  plan->knobs.tile_n = sp.acc_cols; plan->knobs.swizzle_bytes = 128; plan->knobs.stages = sp.ring;
  plan->knobs.acc_stages = 2; plan->knobs.cta_group = 1; plan->knobs.epilogue = 2; plan->knobs.epi_warps = fuse ? hb::kStripFusedEpiWarps : hb::kEpiWarps;
  // the packed-filter wrapper reads these from the GEMM-view parameter block
  plan->p.N = g.CO; plan->p.KW = g.KW; plan->p.CI = g.CI; plan->p.esize_out = eo;
  return HB_OK;
}

// What the NCHW operators add to a conv plan: channel-major output, and an input that is a
// strided view (byte strides of its W, H, N axes) instead of a dense NHWC tensor.
struct ConvExtra {
  bool out_nchw;
  long long w_stride, h_stride, n_stride;
  int kslab;  // > 1: every tile is cut into this many K slices, each stored to its own slab of `out`
  // 3-D convolution: depth extent, taps, stride and padding (D = KD = 1, stride 1, pad 0 otherwise)
  int D, KD, stride_d, pad_d;
};

// pad_h / pad_w: rows / columns of zeros on each side of the height / width axis.  The 2-D
// operators of the reference pad both axes alike; its 1-D convolutions are the H = KH = 1 case
// with pad_h = 0.
int plan_conv(const void* in, const void* w, void* out, int N, int H, int W, int CI, int CO, int KH,
              int KW, int stride_h, int stride_w, int pad_h, int pad_w, int dil_h, int dil_w,
              hb_dtype in_a, hb_dtype in_w, hb_dtype out_t, const hb_knobs* knobs, hb_plan* plan,
              const ConvExtra* ex = nullptr) {
  const bool out_nchw = ex && ex->out_nchw;
  if (N <= 0 || H <= 0 || W <= 0 || CI <= 0 || CO <= 0 || KH <= 0 || KW <= 0) return HB_ERR_SHAPE;
  if (stride_h <= 0 || stride_w <= 0 || dil_h <= 0 || dil_w <= 0 || pad_h < 0 || pad_w < 0) return HB_ERR_SHAPE;
  if (mma_kind(in_a, in_w, out_t) < 0) return HB_ERR_DTYPE;
  const int es = esize(in_a);
  if ((CI * es) % 32 != 0) return HB_ERR_SHAPE;
  if ((static_cast<long long>(CO) * es) % 16 != 0) return HB_ERR_SHAPE;
  // im2col-mode TMA limits: 8-bit signed corners, 8-bit tap offsets, traversal stride <= 8.
  if (pad_h > 127 || pad_w > 127 || (KW - 1) * dil_w > 255 || (KH - 1) * dil_h > 255) return HB_ERR_SHAPE;
  if (pad_w - (KW - 1) * dil_w < -128 || pad_h - (KH - 1) * dil_h < -128) return HB_ERR_SHAPE;
  if (stride_h > 8 || stride_w > 8) return HB_ERR_SHAPE;
  const int HO = conv_out_extent(H, KH, stride_h, pad_h, dil_h);
  const int WO = conv_out_extent(W, KW, stride_w, pad_w, dil_w);
  if (HO <= 0 || WO <= 0) return HB_ERR_SHAPE;
  const int D3 = (ex && ex->D > 0) ? ex->D : 1, KD = (ex && ex->KD > 0) ? ex->KD : 1;
  const int stride_d = (ex && ex->stride_d > 0) ? ex->stride_d : 1, pad_d = ex ? ex->pad_d : 0;
  if (pad_d < 0 || pad_d > 127 || KD - 1 > 255 || pad_d - (KD - 1) < -128 || stride_d > 8) return HB_ERR_SHAPE;
  const int DO = conv_out_extent(D3, KD, stride_d, pad_d, 1);
  if (DO <= 0) return HB_ERR_SHAPE;
  const long long M = static_cast<long long>(N) * DO * HO * WO;
  const long long K = static_cast<long long>(KD) * KH * KW * CI;
  if (M > 0x7fffffffLL || K > 0x7fffffffLL) return HB_ERR_SHAPE;
  if (!in || !w || !out) return HB_ERR_ALIGN;
  if (!aligned16(in) || !aligned16(w) || !aligned16(out)) return HB_ERR_ALIGN;
  Driver& d = driver();
  if (d.status != HB_OK) return d.status;
  Problem pr{2, 1, static_cast<int>(M), CO, static_cast<int>(K), in_a, in_w, out_t, true, CI};
  ConvGeom cg{N, H, W, CI, CO, KH, KW, stride_h, stride_w, pad_h, pad_w, dil_h, dil_w, HO, WO, out_nchw,
              ex ? ex->w_stride : 0, ex ? ex->h_stride : 0, ex ? ex->n_stride : 0, ex ? ex->kslab : 0,
              D3, KD, stride_d, pad_d, DO};
  // only the im2col kernel reads through custom strides or walks a third spatial axis
  const bool strided_view = cg.w_stride > 0 || is_3d(cg);
  const int algo = knobs ? knobs->conv_algo : 0;
  if (algo < 0 || algo > 4 || (algo >= 2 && strided_view)) return HB_ERR_KNOB;
  if (algo == 0 && !strided_view && !out_nchw && in_w == HB_F16 && !(knobs && knobs->silent_producer)) {
    // The strip kernel's fused-row form: picked where it applies and the filter has at least two
    // rows; with a 2-byte output where tiles fill three quarters of the MMA rows, with a 4-byte
    // output up to a padded width of 100.  Measured on a B200, 3x3, 64 -> 64 channels, fp16 out
    // (im2col / strip / wide strip / fused, us): 32 x 56 x 56: 24.2 / 18.7 / 15.5 / 14.2;
    // 64 x 28 x 28: 14.0 / 12.2 / 12.2 / 9.8; 16 x 96 x 96: 31.2 / 26.7 / 20.4 / 18.8;
    // 16 x 112 x 112: 41.6 / 30.6 / 51.4 / 21.2; but 32 x 64 x 64 (half of the MMA rows idle):
    // 27.8 / 32.6 / 18.5 / 21.9 and 16 x 80 x 80: 24.3 / 22.7 / 15.6 / 16.8.  fp32 out:
    // 32 x 56 x 56: 25.4 / 18.0 / 19.7 / 15.1; 16 x 80 x 80: 25.6 / 21.7 / 20.5 / 17.7;
    // 16 x 96 x 96: 32.6 / 25.5 / 38.7 / 20.5; but 16 x 112 x 112: 43.3 / 29.6 / 51.8 / 35.1.
    // A one-row filter is level with the strip kernel.
    hb::StripParams pf;
    std::memset(&pf, 0, sizeof(pf));
    const int eo = esize(out_t);
    const bool fits_f = strip_smem_bytes(cg, es, eo, &pf, true) != 0;
    const bool rows_used = fits_f && static_cast<long long>(HO) * pf.Wp * 4 >= static_cast<long long>(pf.groups) * 128 * 3;
    if (fits_f && KH >= 2 && K * es <= 2048 && (eo == 2 ? rows_used : pf.Wp <= 100)) {
      hb_knobs k0;
      if (knobs) k0 = *knobs; else std::memset(&k0, 0, sizeof(k0));
      k0.conv_algo = 4;
      return build_strip_plan(d, cg, in_a, in_w, out_t, k0, in, w, out, plan);
    }
  }
  {
    // The wide strip kernel (channels on M, 256 positions on N): asked for, or picked when it applies,
    // the filter has more than one tap and the reduction is short enough that operand traffic, not
    // tensor time, bounds the layer (measured on the 56 x 56 x 64 -> 64 layer: 14.6 us against 18.2 us
    // for the strip kernel and 23.8 us for the im2col kernel).  Not picked for padded rows wider
    // than 90 pixels (a strip of 256 positions plus the taps' reach is then many image rows:
    // 16 x 112 x 112 x 64 -> 64 measured 51.4 us against 30.6 us for the strip kernel), nor for
    // 64 output channels with a 4-byte output (19.7 against 18.0 us on the 56 x 56 layer).
    hb_knobs k0;
    if (knobs) k0 = *knobs; else std::memset(&k0, 0, sizeof(k0));
    const bool fits_t = !strided_view && !out_nchw && in_w == HB_F16 && !k0.silent_producer &&
                        strip_t_smem_bytes(cg, in_a, out_t, nullptr, strip_t_max_l(algo == 3 ? k0.tile_n : 0)) != 0;
    const bool wide_pays = W + 2 * pad_w <= 90 && (CO != 64 || esize(out_t) == 2);
    if (algo == 3 && !fits_t) return HB_ERR_KNOB;
    if (algo == 3 || (algo == 0 && fits_t && wide_pays && KH * KW > 1 && K * es <= 2048)) {
      if (algo == 0) k0.tile_n = 0;  // (tile_n is the GEMM kernels' knob unless this kernel was asked for)
      return build_strip_t_plan(d, cg, in_a, in_w, out_t, k0, in, w, out, plan);
    }
  }
  if (algo != 1 && !strided_view) {
    hb::StripParams probe;
    std::memset(&probe, 0, sizeof(probe));
    const bool fits = strip_smem_bytes(cg, es, esize(out_t), &probe) != 0;
    // Picked by default when the filter has more than one tap (so pixels would otherwise be
    // re-fetched per tap), tiles fill at least three quarters of the 128 MMA rows, and the whole
    // reduction is short enough that operand traffic, not tensor time, bounds the kernel.
    const bool rows_used = fits && static_cast<long long>(HO) * probe.Wp * 4 >= static_cast<long long>(probe.groups) * 128 * 3;
    const bool wanted = algo == 2 || (KH * KW > 1 && rows_used && K * es <= 2048);
    if (algo == 2 && !fits) return HB_ERR_KNOB;
    if (algo == 4) {
      if (in_w != HB_F16 || strip_smem_bytes(cg, es, esize(out_t), nullptr, true) == 0) return HB_ERR_KNOB;
      hb_knobs k0 = *knobs;
      return build_strip_plan(d, cg, in_a, in_w, out_t, k0, in, w, out, plan);
    }
    if (fits && wanted) {
      hb_knobs k0;
      if (knobs) k0 = *knobs; else std::memset(&k0, 0, sizeof(k0));
      k0.conv_algo = 2;
      return build_strip_plan(d, cg, in_a, in_w, out_t, k0, in, w, out, plan);
    }
  }
  hb_knobs k;
  if (out_nchw) {
    // channel-major output goes through the direct-store epilogue; split-K's zeroing pass knows
    // only the row-major tile layout
    hb_knobs k0;
    if (knobs) k0 = *knobs; else std::memset(&k0, 0, sizeof(k0));
    k0.epilogue = 2;
    k0.split_k = 1;
    k0.balance = 1;
    resolve_knobs(pr, &k0, d.sm_count, &k);
  } else {
    resolve_knobs(pr, knobs, d.sm_count, &k);
  }
  k.conv_algo = 1;
  return build_plan(d, pr, k, &cg, in, w, out, plan);
}

int plan_conv_packed(const void* in, const void* w_packed, void* out, int N, int H, int W, int CI,
                     int CO, int KH, int KW, int stride_h, int stride_w, int pad_h, int pad_w,
                     int dil_h, int dil_w, int sco, void* scratch, size_t scratch_bytes,
                     const hb_knobs* knobs, hb_plan* plan) {
  if (sco != 64 && sco != 48 && sco != 32) return HB_ERR_SHAPE;
  if (CI <= 0 || CO <= 0 || KH <= 0 || KW <= 0) return HB_ERR_SHAPE;
  if (CI % 4 != 0 || CO % sco != 0) return HB_ERR_SHAPE;
  if (!scratch || scratch_bytes < hb_conv2d_packed_scratch_bytes(CI, CO, KH, KW))
    return HB_ERR_SCRATCH;
  if (!w_packed || !aligned16(w_packed) || !aligned16(scratch)) return HB_ERR_ALIGN;
  const int rc = plan_conv(in, scratch, out, N, H, W, CI, CO, KH, KW, stride_h, stride_w, pad_h, pad_w,
                           dil_h, dil_w, HB_U8, HB_S8, HB_S32, knobs, plan);
  if (rc != HB_OK) return rc;
  const long long groups = static_cast<long long>(KH) * KW * (CI / 4) * CO;
  int blocks = static_cast<int>((groups + 255) / 256);
  const int cap = driver().sm_count * 8;
  if (blocks > cap) blocks = cap;
  plan->packed_w = w_packed;
  plan->scratch = scratch;
  plan->unpack_blocks = blocks;
  plan->sco = sco;
  plan->KH = KH;
  return HB_OK;
}

size_t align256(size_t v) { return (v + 255) & ~static_cast<size_t>(255); }

struct NchwLayout {
  int CIp, HO, WO, DO;
  // few-channel ("stem") form: KWp horizontally adjacent pixels of `cis` channels make one K block
  bool stem;
  int cis, KWp, Hs, Ws, Wv;
  // strided 1x1 conv: the glue keeps only the pixels the conv reads, and the conv runs unstrided
  bool subsample;
  size_t in_bytes, w_bytes, ws_bytes, total;
};

// Most slabs a split-K plan of the NCHW operators takes, and the largest output (elements) it is
// considered for: small outputs are the ones that leave most of the GPU idle.
constexpr int kMaxSlabs = 8;
constexpr long long kSlabMaxOutElems = 1ll << 21;

// Depth axis of the NCDHW operator; {1, 1, 1, 0} for the 2-D and 1-D ones.
struct Depth {
  int D, KD, stride, pad;
};
constexpr Depth kNoDepth{1, 1, 1, 0};

bool nchw_layout(int N, int H, int W, int CI, int CO, int KH, int KW, int sh, int sw, int pad_h,
                 int pad_w, hb_dtype in_a, hb_dtype out_t, NchwLayout* L, const Depth& dz = kNoDepth) {
  const int es = esize(in_a), eo = esize(out_t);
  if (es == 0 || eo == 0 || N <= 0 || H <= 0 || W <= 0 || CI <= 0 || CO <= 0 || KH <= 0 || KW <= 0 ||
      sh <= 0 || sw <= 0 || pad_h < 0 || pad_w < 0 || dz.D <= 0 || dz.KD <= 0 || dz.stride <= 0 || dz.pad < 0)
    return false;
  const bool three_d = dz.D > 1 || dz.KD > 1 || dz.pad > 0;
  L->DO = conv_out_extent(dz.D, dz.KD, dz.stride, dz.pad, 1);
  if (L->DO <= 0) return false;
  const int gran = 32 / es;  // the NHWC kernels want whole 32-byte channel groups
  L->CIp = (CI + gran - 1) / gran * gran;
  L->HO = conv_out_extent(H, KH, sh, pad_h, 1);
  L->WO = conv_out_extent(W, KW, sw, pad_w, 1);
  if (L->HO <= 0 || L->WO <= 0) return false;
  L->subsample = !three_d && KH == 1 && KW == 1 && pad_h == 0 && pad_w == 0 && (sh > 1 || sw > 1);
  const size_t kept_px =
      L->subsample ? static_cast<size_t>(L->HO) * L->WO : static_cast<size_t>(dz.D) * H * W;
  L->in_bytes = align256(static_cast<size_t>(N) * kept_px * L->CIp * es);
  L->w_bytes = align256(static_cast<size_t>(dz.KD) * KH * KW * L->CIp * CO * es);
  // With at most 16 bytes of channels per pixel and a filter row of 2..8 taps, a whole filter
  // row fits one 64- or 128-byte K block: far fewer, fuller pipeline stages than one tap each.
  L->cis = 16 / es;
  L->stem = !three_d && CI <= L->cis && KW >= 2 && KW <= 8;
  if (L->stem) {
    L->KWp = KW <= 4 ? 4 : 8;
    L->Hs = (L->HO - 1) * sh + KH;           // rows the windows touch, borders included
    L->Wv = (L->WO - 1) * sw + 1;            // window start positions along a row
    L->Ws = (L->WO - 1) * sw + L->KWp;       // pixels per stored row
    L->in_bytes = align256(static_cast<size_t>(N) * L->Hs * L->Ws * 16);
    L->w_bytes = align256(static_cast<size_t>(KH) * L->KWp * 16 * CO);
  }
  // room for the partial sums of a split-K plan (4-byte accumulators, row-major (M, CO) slabs)
  const long long out_elems = static_cast<long long>(N) * L->DO * L->HO * L->WO * CO;
  L->ws_bytes = out_elems <= kSlabMaxOutElems ? align256(static_cast<size_t>(out_elems) * 4 * kMaxSlabs) : 0;
  L->total = L->in_bytes + L->w_bytes + L->ws_bytes;
  return true;
}

int plan_conv_nchw(const void* in, const void* w, void* out, int N, int H, int W, int CI, int CO,
                   int KH, int KW, int sh, int sw, int pad_h, int pad_w, hb_dtype in_a, hb_dtype in_w,
                   hb_dtype out_t, void* scratch, size_t scratch_bytes, const hb_knobs* knobs,
                   hb_plan* plan, const Depth& dz = kNoDepth) {
  NchwLayout L;
  if (!nchw_layout(N, H, W, CI, CO, KH, KW, sh, sw, pad_h, pad_w, in_a, out_t, &L, dz)) return HB_ERR_SHAPE;
  if (esize(in_w) != esize(in_a)) return HB_ERR_DTYPE;
  if (!scratch || scratch_bytes < L.total) return HB_ERR_SCRATCH;
  if (!in || !w || !out) return HB_ERR_ALIGN;
  if ((reinterpret_cast<uintptr_t>(scratch) & 255u) != 0) return HB_ERR_ALIGN;
  // A 1x1, stride-1, unpadded conv is, per image, out (CO x P) = filter (CO x CI) . in (CI x P): a
  // batched GEMM on the NCHW tensors as they are (filter as the shared K-major A, each image as an
  // N-contiguous B, row-major C = NCHW), with no layout pass.  Needs 16-byte rows for the tensor maps.
  const long long P1 = static_cast<long long>(dz.D) * H * W;
  const int es1 = esize(in_a), eo1 = esize(out_t);
  if (KH == 1 && KW == 1 && sh == 1 && sw == 1 && pad_h == 0 && pad_w == 0 && dz.KD == 1 && dz.stride == 1 &&
      dz.pad == 0 && (P1 * es1) % 16 == 0 &&
      (static_cast<long long>(CI) * es1) % 16 == 0 && P1 <= 0x7fffffffLL && P1 >= 32 &&
      aligned16(in) && aligned16(w) && aligned16(out) && (!knobs || knobs->conv_algo == 0)) {
    if (mma_kind(in_w, in_a, out_t) < 0) return HB_ERR_DTYPE;
    Driver& d = driver();
    if (d.status != HB_OK) return d.status;
    Problem pr{1, N, CO, static_cast<int>(P1), CI, in_w, in_a, out_t, false, 0, 0, true};
    hb_knobs k0, k;
    if (knobs) k0 = *knobs; else std::memset(&k0, 0, sizeof(k0));
    if (k0.epilogue == 0 && (P1 * eo1) % 16 != 0) k0.epilogue = 2;
    if (k0.epilogue == 1 && (P1 * eo1) % 16 != 0) return HB_ERR_KNOB;
    k0.l2_prefetch = -1;
    resolve_knobs(pr, &k0, d.sm_count, &k);
    return build_plan(d, pr, k, nullptr, w, in, out, plan);
  }
  uint8_t* s_in = static_cast<uint8_t*>(scratch);
  uint8_t* s_w = s_in + L.in_bytes;
  if (!aligned16(out)) return HB_ERR_ALIGN;
  const int es = esize(in_a);
  uint8_t* s_ws = s_w + L.w_bytes;
  // The conv the kernel runs: the NHWC form of the problem, or its few-channel form.
  ConvExtra ex{true, 0, 0, 0, 0, dz.D, dz.KD, dz.stride, dz.pad};
  int cH = H, cW = W, cCI = L.CIp, cKW = KW, cpad_h = pad_h, cpad_w = pad_w, csh = sh, csw = sw;
  if (L.subsample) { cH = L.HO; cW = L.WO; csh = 1; csw = 1; }
  if (L.stem) {
    const long long px = 16;  // bytes per stored pixel
    ex.w_stride = px; ex.h_stride = px * L.Ws; ex.n_stride = px * L.Ws * L.Hs;
    cH = L.Hs; cW = L.Wv; cCI = L.KWp * L.cis; cKW = 1; cpad_h = 0; cpad_w = 0;
  }
  int rc = plan_conv(s_in, s_w, out, N, cH, cW, cCI, CO, KH, cKW, csh, csw, cpad_h, cpad_w, 1, 1, in_a, in_w,
                     out_t, knobs, plan, &ex);
  if (rc != HB_OK) return rc;
  // A problem with far fewer tiles than SMs and a long reduction runs as split-K: every tile's K
  // range is cut into slabs stored side by side in the workspace, and a small kernel adds them in
  // slab order while it writes NCHW (deterministic, no atomics, any output type).
  bool post = false;
  int slabs = 0;
  if (!plan->strip && L.ws_bytes > 0 && (!knobs || knobs->split_k != 1)) {
    const int units = driver().sm_count / plan->knobs.cta_group;
    const int tiles = plan->p.num_tiles;
    slabs = tiles > 0 ? units / tiles : 0;
    if (knobs && knobs->split_k > 1) slabs = knobs->split_k;
    if (slabs > kMaxSlabs) slabs = kMaxSlabs;
    while (slabs > 1 && plan->p.num_kb / slabs < 4) --slabs;
    // the extra launch and the workspace round trip cost about 4 us; a K block of the im2col conv
    // takes about 0.5 us
    post = slabs >= 2 && ((knobs && knobs->split_k > 1) ||
                          static_cast<long long>(plan->p.num_kb) * (slabs - 1) >= 16ll * slabs);
  }
  if (post) {
    const hb_dtype acc_t = (in_a == HB_F16) ? HB_F32 : HB_S32;
    ex.out_nchw = false;
    ex.kslab = slabs;
    hb_knobs k0;
    if (knobs) k0 = *knobs; else std::memset(&k0, 0, sizeof(k0));
    k0.epilogue = 0;
    k0.split_k = 0;
    k0.tail_split = 1;
    k0.balance = 1;  // the slabs are this plan's split
    if (k0.tile_n != 0 && out_t == HB_F16 && k0.tile_n % 64 != 0) k0.tile_n = 0;
    rc = plan_conv(s_in, s_w, s_ws, N, cH, cW, cCI, CO, KH, cKW, csh, csw, cpad_h, cpad_w, 1, 1, in_a, in_w,
                   acc_t, &k0, plan, &ex);
    if (rc != HB_OK) return rc;
    plan->has_post = true;
    plan->post_ws = s_ws; plan->post_out = out;
    plan->post_slabs = slabs; plan->post_P = L.DO * L.HO * L.WO; plan->post_CO = CO; plan->post_N = N;
    plan->post_slab_elems = static_cast<long long>(N) * L.DO * L.HO * L.WO * CO;
    plan->post_kind = out_t == HB_F16 ? 0 : (out_t == HB_F32 ? 1 : 2);
  }
  if (L.stem) {
    hb::StemPre& g = plan->stem;
    g.in = in; g.in_t = s_in; g.w = w; g.w_t = s_w;
    g.N = N; g.CI = CI; g.H = H; g.W = W; g.CO = CO; g.KH = KH; g.KW = KW; g.KWp = L.KWp; g.cis = L.cis;
    g.Hs = L.Hs; g.Ws = L.Ws; g.pad_h = pad_h; g.pad_w = pad_w;
    g.in_px = static_cast<long long>(N) * L.Hs * L.Ws;
    g.w_elems = static_cast<long long>(KH) * L.KWp * L.cis * CO;
    long long blocks = (g.in_px + 255) / 256;
    const long long cap = static_cast<long long>(driver().sm_count) * 16;
    if (blocks > cap) blocks = cap;
    plan->pre_grid = static_cast<int>(blocks);
    plan->pre_esize = es;
    plan->pre_is_stem = true;
    plan->has_pre = true;
    return HB_OK;
  }
  const int T = dz.KD * KH * KW, P = L.subsample ? L.HO * L.WO : dz.D * H * W;
  const int vec = 8 / es, tile = 16 * vec;
  hb::NchwPre& g = plan->pre;
  g.in = in; g.in_t = s_in; g.w = w; g.w_t = s_w;
  g.N = N; g.CI = CI; g.CIp = L.CIp; g.P = P; g.CO = CO; g.T = T;
  g.sub_wo = 0; g.sub_col = 1; g.sub_row = 0; g.src_P = H * W;
  if (L.subsample) { g.sub_wo = L.WO; g.sub_col = sw; g.sub_row = sh * W; }
  // 8-byte accesses need every image and channel row of the source to start on 8 bytes
  g.vec = (!L.subsample && P % vec == 0 && (reinterpret_cast<uintptr_t>(in) & 7u) == 0) ? 1 : 0;
  g.in_bx = (P + tile - 1) / tile;
  g.in_by = (L.CIp + tile - 1) / tile;
  const long long in_blocks = static_cast<long long>(g.in_bx) * g.in_by * N;
  g.f_tchunk = T < hb::kFilterRun ? T : hb::kFilterRun;
  g.f_ci_tile = hb::kFilterRun / g.f_tchunk;
  if (g.f_ci_tile > 32) g.f_ci_tile = 32;
  g.f_bco = (CO + 31) / 32;
  g.f_bci = (L.CIp + g.f_ci_tile - 1) / g.f_ci_tile;
  g.f_bt = (T + g.f_tchunk - 1) / g.f_tchunk;
  if (T == 1) {
    // a plain (CO x CI) -> (CIp x CO) transpose: the tile transposer, vectorised when it may be
    g.f_bco = (CO + tile - 1) / tile;
    g.f_bci = (L.CIp + tile - 1) / tile;
    g.f_vec = (CI % vec == 0 && CO % vec == 0 && (reinterpret_cast<uintptr_t>(w) & 7u) == 0) ? 1 : 0;
  }
  const long long f_blocks = static_cast<long long>(g.f_bco) * g.f_bci * g.f_bt;
  if (in_blocks + f_blocks > 0x7fffffffLL) return HB_ERR_SHAPE;
  g.in_blocks = static_cast<int>(in_blocks);
  plan->pre_grid = static_cast<int>(in_blocks + f_blocks);
  plan->pre_esize = es;
  plan->has_pre = true;
  return HB_OK;
}
}  // namespace
