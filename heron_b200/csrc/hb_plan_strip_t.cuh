// Plan of the wide strip conv kernel (hb_conv_strip_t.cuh): geometry, shared-memory budget,
// tensor maps.
#pragma once
#include "hb_host.cuh"
#include "hb_conv_strip_t.cuh"

namespace {

// Shared-memory need of the wide strip algorithm for a geometry, or 0 when it does not apply:
// stride 1, fp16, whole 128-byte channel chunks, 64 or 128 output channels (the MMA's M), and the
// filter plus two strips within shared memory.
int strip_t_smem_bytes(const ConvGeom& g, hb_dtype in_a, hb_dtype out_t, hb::StripTParams* sp, int max_l = 256) {
  if (in_a != HB_F16 || (out_t != HB_F16 && out_t != HB_F32)) return 0;
  if (g.stride_h != 1 || g.stride_w != 1 || g.out_nchw || g.w_stride > 0 || is_3d(g)) return 0;
  if ((g.CI * 2) % 128 != 0) return 0;
  if (g.CO != 64 && g.CO != 128) return 0;
  const int Wp = g.W + 2 * g.pad_w;
  if (Wp < 1 || Wp > 256) return 0;
  const int P = (g.HO - 1) * Wp + g.WO;
  const int max_off = (g.KH - 1) * g.dil_h * Wp + (g.KW - 1) * g.dil_w;
  const int n_cchunks = g.CI * 2 / 128;
  const long long filt = static_cast<long long>(g.KH) * g.KW * g.CI * g.CO * 2;
  // Tiles of 256 positions where the filter, two strips and the epilogue's staging buffer (one
  // tile of output) fit shared memory, else narrower ones.
  int L = 0, SR = 0, strip_bytes = 0;
  long long smem = 0;
  if (max_l < 64 || max_l > 256 || max_l % 64 != 0) return 0;
  for (int cand = max_l; cand >= 64; cand -= 64) {
    L = cand;
    if (P < L) L = (P + 15) & ~15;
    // rows a strip must hold: a tile may start at any column, reads L positions and the taps
    SR = (Wp - 1 + L + max_off + Wp - 1) / Wp;
    strip_bytes = (SR * Wp * 128 + 1023) & ~1023;
    const long long stage = static_cast<long long>(L) * g.CO * esize(out_t);
    smem = ((filt + 1023) & ~1023LL) + 2LL * n_cchunks * strip_bytes + stage + 1024 + 512;
    if (SR <= 256 && smem <= kSmemLimit) break;
    smem = 0;
  }
  if (smem == 0) return 0;
  int ring = 2;
  while (ring < hb::kMaxStripTRing && smem + static_cast<long long>(n_cchunks) * strip_bytes <= kSmemLimit) {
    smem += static_cast<long long>(n_cchunks) * strip_bytes;
    ++ring;
  }
  if (sp) {
    sp->Wp = Wp; sp->P = P; sp->L = L; sp->SR = SR; sp->strip_bytes = strip_bytes; sp->n_cchunks = n_cchunks;
    sp->tiles_per_img = (P + L - 1) / L;
    sp->ring = ring;
  }
  return static_cast<int>(smem);
}

// The positions per tile the knob tile_n asks of the wide strip kernel: a multiple of 64 between
// 64 and 256 (the knob's own grid is multiples of 32: those round down), 256 when unset.
int strip_t_max_l(int tile_n) {
  if (tile_n <= 0) return 256;
  const int l = tile_n / 64 * 64;
  return l < 64 ? 64 : (l > 256 ? 256 : l);
}

int build_strip_t_plan(Driver& d, const ConvGeom& g, hb_dtype in_a, hb_dtype in_w, hb_dtype out_t,
                       const hb_knobs& k, const void* in, const void* w, void* out, hb_plan* plan) {
  if (g_plan_owns_flags) release_split_flags(plan->p.flags, plan->owned_flags);
  std::memset(plan, 0, sizeof(*plan));
  hb::StripTParams& sp = plan->spt;
  // (knob tile_n caps the positions per tile: 64, 128, 192 or 256)
  const int smem = strip_t_smem_bytes(g, in_a, out_t, &sp, strip_t_max_l(k.tile_n));
  if (smem == 0 || in_w != HB_F16) return HB_ERR_KNOB;
  const long long tiles = static_cast<long long>(g.N) * sp.tiles_per_img;
  if (tiles > 0x7fffffffLL) return HB_ERR_SHAPE;
  sp.N = g.N; sp.H = g.H; sp.W = g.W; sp.CI = g.CI; sp.CO = g.CO; sp.KH = g.KH; sp.KW = g.KW;
  sp.pad_h = g.pad_h; sp.pad_w = g.pad_w; sp.dil_h = g.dil_h; sp.dil_w = g.dil_w; sp.HO = g.HO; sp.WO = g.WO;
  sp.num_tiles = static_cast<int>(tiles);
  sp.esize_out = esize(out_t);
  sp.tmem_cols = 512;  // two accumulators of up to 256 positions
  // fp32 accumulate, fp16 operands, A (the filter) MN-major, B (the strip) K-major, M = CO; the
  // kernel adds each tile's N
  uint32_t idesc = 1u << 4;
  idesc |= 1u << 15;
  idesc |= static_cast<uint32_t>(g.CO >> 4) << 24;
  sp.idesc = idesc;
  sp.out = out;
  sp.probe = k.probe;
  if (k.silent_producer) return HB_ERR_KNOB;  // (that test hook lives in the GEMM kernel)
  // input as a tiled (C, W, H, N) tensor: one box = 128 bytes of channels x padded width x strip rows
  cuuint64_t dims[4] = {static_cast<cuuint64_t>(g.CI), static_cast<cuuint64_t>(g.W),
                        static_cast<cuuint64_t>(g.H), static_cast<cuuint64_t>(g.N)};
  cuuint64_t strides[3] = {static_cast<cuuint64_t>(g.CI) * 2, static_cast<cuuint64_t>(g.W) * g.CI * 2,
                           static_cast<cuuint64_t>(g.H) * g.W * g.CI * 2};
  cuuint32_t box[4] = {64u, static_cast<cuuint32_t>(sp.Wp), static_cast<cuuint32_t>(sp.SR), 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = d.tiled(&plan->tmA, tmap_dtype(in_a), 4, const_cast<void*>(in), dims, strides, box, estr,
                       CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                       CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return HB_ERR_LAUNCH;
  const long long K = static_cast<long long>(g.KH) * g.KW * g.CI;
  const uint64_t rowB = static_cast<uint64_t>(g.CO) * 2;
  int rc = encode_tiled3(d, &plan->tmB, in_w, w, g.CO, K, 1, rowB, rowB * K, 64, 64, 128);
  if (rc != HB_OK) return rc;
  int grid = d.sm_count;
  if (k.max_ctas > 0 && k.max_ctas < grid) grid = k.max_ctas;
  if (sp.num_tiles < grid) grid = sp.num_tiles;
  plan->strip_t = true;
  plan->grid = grid;
  plan->smem = smem;
  plan->knobs = k;
  plan->knobs.conv_algo = 3;
  // fields hb_plan_knobs reports
  plan->knobs.tile_n = sp.L; plan->knobs.swizzle_bytes = 128; plan->knobs.stages = sp.ring;
  plan->knobs.acc_stages = 2; plan->knobs.cta_group = 1; plan->knobs.epilogue = 2;
  plan->knobs.epi_warps = hb::kWideEpiWarps; plan->knobs.balance = 1; plan->knobs.split_k = 1; plan->knobs.tail_split = 1; plan->knobs.k_slices = 1;
  plan->p.N = g.CO; plan->p.KW = g.KW; plan->p.CI = g.CI; plan->p.esize_out = sp.esize_out;
  return HB_OK;
}

}  // namespace
