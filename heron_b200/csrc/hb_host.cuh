// Host-side foundations of libheron_b200.so: driver entry points, dtype and descriptor helpers,
// the problem description, knob defaults and limits, and the plan object.
//
// Nothing in the library allocates device memory: the kernels work on the caller's buffers, the
// tensor maps travel as kernel parameters, and the device status word is a __device__ variable.
#pragma once
#include "../../include/heron_b200.h"
#include "hb_kernel.cuh"
#include "hb_glue.cuh"
#include "hb_conv_strip.cuh"
#include "hb_conv_strip_t.cuh"

#include <cuda.h>
#include <cuda_runtime.h>
#include <cstdio>
#include <cstring>
#include <mutex>
#include <new>

namespace {

using hb::KParams;

constexpr int kSmemLimit = 232448;  // 227 KiB opt-in dynamic shared memory per CTA on sm_100
constexpr int kSmemSlack = 2048 /*alignment of the ring and of the epilogue staging*/ + 512 /*barriers*/;

// ---- driver entry points (no link-time dependency on libcuda) -------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
typedef CUresult (*EncodeIm2colFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                   const cuuint64_t*, const cuuint64_t*, const int*, const int*,
                                   cuuint32_t, cuuint32_t, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion,
                                   CUtensorMapFloatOOBfill);

struct Driver {
  EncodeTiledFn tiled = nullptr;
  EncodeIm2colFn im2col = nullptr;
  int sm_count = 0;
  int driver_version = 0;
  int status = HB_ERR_DEVICE;
};

// Per-device set-up (kernel attributes are per device): done the first time a device is current
// when an entry point runs.  Driver entry points are process-wide.
constexpr int kMaxDev = 64;

bool setup_device(Driver* d) {
  cudaDeviceProp prop;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return false;
  if (cudaGetDeviceProperties(&prop, dev) != cudaSuccess) return false;
  if (prop.major != 10) return false;
  d->sm_count = prop.multiProcessorCount;
  // Opt in to the large dynamic shared-memory carve-out for every kernel instantiation.
  const void* kernels[31] = {
      reinterpret_cast<const void*>(&hb::hb_conv_strip_t_kernel<2>),
      reinterpret_cast<const void*>(&hb::hb_conv_strip_t_kernel<4>),
      reinterpret_cast<const void*>(&hb::hb_umma_kernel<4, 1, 0, 1>),
      reinterpret_cast<const void*>(&hb::hb_umma_kernel<2, 1, 0, 1>),
      reinterpret_cast<const void*>(&hb::hb_umma_kernel<4, 1, 1, 1>),
      reinterpret_cast<const void*>(&hb::hb_umma_kernel<4, 2, 0, 1>),
      reinterpret_cast<const void*>(&hb::hb_umma_kernel<2, 2, 0, 1>),
      reinterpret_cast<const void*>(&hb::hb_umma_kernel<4, 2, 1, 1>),
      reinterpret_cast<const void*>(&hb::hb_umma_kernel<4, 1, 0, 2>),
      reinterpret_cast<const void*>(&hb::hb_umma_kernel<2, 1, 0, 2>),
      reinterpret_cast<const void*>(&hb::hb_umma_kernel<4, 1, 1, 2>),
      reinterpret_cast<const void*>(&hb::hb_umma_kernel<4, 2, 0, 2>),
      reinterpret_cast<const void*>(&hb::hb_umma_kernel<2, 2, 0, 2>),
      reinterpret_cast<const void*>(&hb::hb_umma_kernel<4, 2, 1, 2>),
      reinterpret_cast<const void*>(&hb::hb_umma_kernel<4, 1, 0, 1, 8>),
      reinterpret_cast<const void*>(&hb::hb_umma_kernel<2, 1, 0, 1, 8>),
      reinterpret_cast<const void*>(&hb::hb_umma_kernel<4, 1, 1, 1, 8>),
      reinterpret_cast<const void*>(&hb::hb_umma_kernel<4, 2, 0, 1, 8>),
      reinterpret_cast<const void*>(&hb::hb_umma_kernel<2, 2, 0, 1, 8>),
      reinterpret_cast<const void*>(&hb::hb_umma_kernel<4, 2, 1, 1, 8>),
      reinterpret_cast<const void*>(&hb::hb_umma_kernel<4, 1, 0, 2, 8>),
      reinterpret_cast<const void*>(&hb::hb_umma_kernel<2, 1, 0, 2, 8>),
      reinterpret_cast<const void*>(&hb::hb_umma_kernel<4, 1, 1, 2, 8>),
      reinterpret_cast<const void*>(&hb::hb_umma_kernel<4, 2, 0, 2, 8>),
      reinterpret_cast<const void*>(&hb::hb_umma_kernel<2, 2, 0, 2, 8>),
      reinterpret_cast<const void*>(&hb::hb_umma_kernel<4, 2, 1, 2, 8>),
      reinterpret_cast<const void*>(&hb::hb_conv_strip_kernel<4, 0>),
      reinterpret_cast<const void*>(&hb::hb_conv_strip_kernel<2, 0>),
      reinterpret_cast<const void*>(&hb::hb_conv_strip_kernel<4, 1>),
      reinterpret_cast<const void*>(&hb::hb_conv_strip_kernel<4, 0, 1>),
      reinterpret_cast<const void*>(&hb::hb_conv_strip_kernel<2, 0, 1>)};
  for (const void* k : kernels)
    if (cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemLimit) != cudaSuccess)
      return false;
  return true;
}

Driver& driver() {
  static Driver per_device[kMaxDev];
  static bool tried[kMaxDev] = {false};
  static Driver none;  // status HB_ERR_DEVICE
  static std::mutex mu;
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDev) {
    cudaGetLastError();
    return none;
  }
  std::lock_guard<std::mutex> lock(mu);
  Driver& d = per_device[dev];
  if (tried[dev]) return d;
  tried[dev] = true;
  if (!setup_device(&d)) {
    cudaGetLastError();
    return d;
  }
  cudaDriverGetVersion(&d.driver_version);
  void* fn = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q) != cudaSuccess ||
      q != cudaDriverEntryPointSuccess || fn == nullptr)
    return d;
  d.tiled = reinterpret_cast<EncodeTiledFn>(fn);
  fn = nullptr;
  if (cudaGetDriverEntryPoint("cuTensorMapEncodeIm2col", &fn, cudaEnableDefault, &q) != cudaSuccess ||
      q != cudaDriverEntryPointSuccess || fn == nullptr)
    return d;
  d.im2col = reinterpret_cast<EncodeIm2colFn>(fn);
  d.status = HB_OK;
  return d;
}

int esize(hb_dtype t) {
  switch (t) {
    case HB_F16: return 2;
    case HB_F32: return 4;
    case HB_S8: return 1;
    case HB_U8: return 1;
    case HB_S32: return 4;
  }
  return 0;
}

bool is_i8(hb_dtype t) { return t == HB_S8 || t == HB_U8; }

// 0: fp16 kind, 1: int8 kind, -1: unsupported combination.
int mma_kind(hb_dtype a, hb_dtype b, hb_dtype out) {
  if (a == HB_F16 && b == HB_F16 && (out == HB_F32 || out == HB_F16)) return 0;
  if (is_i8(a) && is_i8(b) && out == HB_S32) return 1;
  return -1;
}

CUtensorMapSwizzle swizzle_enum(int sw) {
  return sw == 128 ? CU_TENSOR_MAP_SWIZZLE_128B
                   : (sw == 64 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_32B);
}

CUtensorMapDataType tmap_dtype(hb_dtype t) {
  switch (t) {
    case HB_F16: return CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    case HB_F32: return CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
    case HB_S32: return CU_TENSOR_MAP_DATA_TYPE_INT32;
    default: return CU_TENSOR_MAP_DATA_TYPE_UINT8;
  }
}

int next_pow2_cols(int c) {
  int p = 32;
  while (p < c) p <<= 1;
  return p;
}

// Instruction descriptor of tcgen05.mma (32 bit): accumulator format bits 4..5, A/B formats bits
// 7..9 / 10..12, A/B major bits 15/16, N/8 in bits 17..22, M/16 in bits 24..28.
uint32_t make_idesc(int kind, hb_dtype a, hb_dtype b, int tile_m, int tile_n, bool b_mn_major) {
  uint32_t d = 0;
  if (kind == 0) {
    d |= 1u << 4;  // fp32 accumulator; A and B formats 0 = fp16
  } else {
    d |= 2u << 4;  // s32 accumulator
    d |= (a == HB_S8 ? 1u : 0u) << 7;
    d |= (b == HB_S8 ? 1u : 0u) << 10;
  }
  d |= 0u << 15;                       // A is K-major
  d |= (b_mn_major ? 1u : 0u) << 16;   // B major
  d |= static_cast<uint32_t>(tile_n >> 3) << 17;
  d |= static_cast<uint32_t>(tile_m >> 4) << 24;
  return d;
}

struct Problem {
  int op;  // 0 gemm, 1 bmm, 2 conv
  int batch, M, N, K;
  hb_dtype in_a, in_b, out;
  bool conv;
  int CI;      // conv only
  int b_rows;  // gemm only: rows B really has when fewer than N (the rest read as zeros); 0 = N
  // bmm only: A (M, K) is shared by all batches and B is stored (batch, K, N) with N contiguous.
  // A 1x1 stride-1 NCHW conv is exactly this product on the tensors as they are:
  // out[n] (CO x P) = filter (CO x CI) . in[n] (CI x P).
  bool shared_a_b_mn;
};

// B is read as (K, N) tiles with N contiguous: the conv filter (HWIO) and the form above.
bool b_mn_major(const Problem& pr) { return pr.conv || pr.shared_a_b_mn; }

// Ring-stage bytes of one CTA: 128 rows of A plus this CTA's share of B's tile_n rows.
int stage_bytes(int tile_n, int sw, int cg) { return (hb::kTileM + tile_n / cg) * sw; }

// Resolves zeros in *in to defaults for this problem.
void resolve_knobs(const Problem& pr, const hb_knobs* in, int sm_count, hb_knobs* out) {
  hb_knobs k;
  if (in) k = *in; else std::memset(&k, 0, sizeof(k));
  const int es = esize(pr.in_a), eo = esize(pr.out);
  const int sms = sm_count > 0 ? sm_count : 148;
  if (k.swizzle_bytes == 0) {
    // Largest swizzle span that divides the K extent of a block: all of K for GEMM (the tail is
    // zero-filled), the channel count for conv (a block never straddles two filter taps).
    k.swizzle_bytes = 128;
    if (pr.conv) {
      const int cbytes = pr.CI * es;
      k.swizzle_bytes = (cbytes % 128 == 0) ? 128 : ((cbytes % 64 == 0) ? 64 : 32);
    } else if (static_cast<long long>(pr.K) * es < 128) {
      const int kbytes = pr.K * es;
      k.swizzle_bytes = kbytes > 64 ? 128 : (kbytes > 32 ? 64 : 32);
    }
  }
  if (k.cta_group == 0) {
    // CTA pairs pay off when the K loop is long enough to amortise the cross-CTA hand-offs of a
    // tile and when each CTA of the pair still gets a whole B chunk of a tile no wider than N.
    const int sw = k.swizzle_bytes ? k.swizzle_bytes : 128;
    const long long kblocks = (static_cast<long long>(pr.K) * es + sw - 1) / sw;
    const int min_pair_n = b_mn_major(pr) ? 2 * sw / es : 64;
    // (on-device tuning of the ResNet-50 and BERT tables picked single CTAs up to 16 K blocks and
    // pairs from 32 on, except for wide outputs, where halving each CTA's share of B pays at once)
    const bool long_k = kblocks >= 24 || (kblocks >= 8 && pr.N >= 1024);
    k.cta_group = (pr.M > hb::kTileM && long_k && pr.N >= min_pair_n) ? 2 : 1;
  }
  if (k.epilogue == 0) {
    // Default: TMA store whenever the output rows are 16-byte multiples.
    k.epilogue = ((static_cast<long long>(pr.N) * eo) % 16 == 0) ? 1 : 2;
  }
  if (k.tile_n == 0) {
    const int step = (eo == 2) ? 64 : 32;
    // MN-major B needs whole swizzle-span chunks of columns in every CTA of the group
    const int chunk = b_mn_major(pr) ? k.cta_group * k.swizzle_bytes / es : step;
    const int gran = chunk > step ? chunk : step;
    const int rows = hb::kTileM * k.cta_group;
    const long long tiles_m = (pr.M + rows - 1) / rows;
    const int units = sms / k.cta_group;
    long long best_cost = -1;
    int best = gran;
    for (int bn = gran; bn <= 256; bn += gran) {
      const long long tiles = tiles_m * ((pr.N + bn - 1) / bn) * pr.batch;
      const long long waves = (tiles + units - 1) / units;
      // operand bytes a CTA pulls per tile
      const long long cost = waves * (hb::kTileM + bn / k.cta_group);
      if (best_cost < 0 || cost < best_cost || (cost == best_cost && bn > best)) {
        best_cost = cost;
        best = bn;
      }
    }
    k.tile_n = best;
  }
  if (k.acc_stages == 0) k.acc_stages = (2 * k.tile_n <= 512) ? 2 : 1;
  if (k.k_slices == 0) {
    // Two swizzle spans of K behind one barrier halve what the MMA thread and the producers spend
    // per span on waits, fences and commits.  Measured on a B200: a gain from 8 spans per tile on
    // if the ring still holds three such stages (4096^3 fp16 in CTA pairs +3 %, int8 +10 %, tiles
    // of 64 or 128 columns +25..38 %), a loss with two (4096^3 in single CTAs -9 %, BERT's
    // 512 x 768 x 768 -14 %) or with 4 spans.
    const int sw = k.swizzle_bytes;
    const long long kblocks = (static_cast<long long>(pr.K) * es + sw - 1) / sw;
    const int epi = k.epilogue == 1 ? hb::kUmmaEpiBytes : 0;
    const int wide = 2 * stage_bytes(k.tile_n, k.swizzle_bytes, k.cta_group);
    const int want = k.stages > 0 ? k.stages : 3;
    k.k_slices = (kblocks >= 8 && want * wide + epi + kSmemSlack <= kSmemLimit) ? 2 : 1;
  }
  if (k.stages == 0) {
    const int epi = k.epilogue == 1 ? hb::kUmmaEpiBytes : 0;
    int s = (kSmemLimit - kSmemSlack - epi) / (k.k_slices * stage_bytes(k.tile_n, k.swizzle_bytes, k.cta_group));
    if (s > 8) s = 8;
    if (s < 1) s = 1;
    k.stages = s;
  }
  if (k.epi_warps == 0) {
    // Eight epilogue warps where a tile's K loop is shorter than its drain (fewer swizzle spans of
    // K than 128-byte column chunks of output: the MMA warp then waits for TMEM), if that leaves
    // each warp at least two chunks.  Measured on a B200 (four warps against eight): 192 batches of
    // 512 x 512 x 64 int8 -> s32 40.3 against 38.7 us, 24 batches 9.25 against 8.85 us; long-K
    // shapes are level or lose up to 0.5 % with eight (4096^3 fp16 108.2 against 108.8 us, the
    // 512-channel 3x3 int8 conv over 1024 images 89.0 against 89.3 us), so they keep four.
    const long long spans = (static_cast<long long>(pr.K) * es + k.swizzle_bytes - 1) / k.swizzle_bytes;
    const int chunks = k.tile_n * eo / 128;
    k.epi_warps = (chunks >= 4 && spans < chunks) ? 8 : 4;
  }
  if (k.l2_prefetch == 0) k.l2_prefetch = -1;
  *out = k;
}

int check_knobs(const Problem& pr, const hb_knobs& k, int* smem_bytes, int* tmem_cols) {
  const int es = esize(pr.in_a), eo = esize(pr.out);
  if (k.swizzle_bytes != 32 && k.swizzle_bytes != 64 && k.swizzle_bytes != 128) return HB_ERR_KNOB;
  const int step = (eo == 2) ? 64 : 32;
  if (k.tile_n < step || k.tile_n > 256 || k.tile_n % step != 0) return HB_ERR_KNOB;
  if (k.stages < 1 || k.stages > hb::kMaxStages) return HB_ERR_KNOB;
  if (k.acc_stages < 1 || k.acc_stages > 2) return HB_ERR_KNOB;
  if (k.acc_stages * k.tile_n > 512) return HB_ERR_KNOB;
  if (k.raster != 0 && k.raster != 1) return HB_ERR_KNOB;
  if (k.epilogue != 1 && k.epilogue != 2) return HB_ERR_KNOB;
  if (k.epilogue == 1 && (static_cast<long long>(pr.N) * eo) % 16 != 0) return HB_ERR_KNOB;
  if (k.max_ctas < 0) return HB_ERR_KNOB;
  if (k.cta_group != 1 && k.cta_group != 2) return HB_ERR_KNOB;
  if (k.l2_prefetch < -1 || k.l2_prefetch > 64) return HB_ERR_KNOB;
  if (k.tail_split != 0 && k.tail_split != 1 && k.tail_split != 2 && k.tail_split != 4) return HB_ERR_KNOB;
  if (k.split_k < 0 || k.split_k > 4) return HB_ERR_KNOB;
  if (k.split_k > 1) {
    // slices add into the output, one after the other: 4-byte elements only
    if (eo != 4 || k.tail_split > 1) return HB_ERR_KNOB;
  }
  if (pr.conv && (pr.CI * es) % k.swizzle_bytes != 0) return HB_ERR_KNOB;
  // whole MN-major chunks in every CTA of the group
  if (b_mn_major(pr) && (k.tile_n / k.cta_group * es) % k.swizzle_bytes != 0) return HB_ERR_KNOB;
  const int epi = k.epilogue == 1 ? hb::kUmmaEpiBytes : 0;
  if (k.k_slices != 1 && k.k_slices != 2) return HB_ERR_KNOB;
  if (k.epi_warps != 4 && k.epi_warps != 8) return HB_ERR_KNOB;
  if (k.balance < 0 || k.balance > 2) return HB_ERR_KNOB;
  if (k.balance == 2 && eo != 4) return HB_ERR_KNOB;  // partial sums travel through the output
  const int smem = k.stages * k.k_slices * stage_bytes(k.tile_n, k.swizzle_bytes, k.cta_group) + epi + kSmemSlack;
  if (smem > kSmemLimit) return HB_ERR_KNOB;
  if (smem_bytes) *smem_bytes = smem;
  if (tmem_cols) *tmem_cols = next_pow2_cols(k.acc_stages * k.tile_n);
  return HB_OK;
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

int encode_tiled3(Driver& d, CUtensorMap* m, hb_dtype t, const void* ptr, uint64_t d0, uint64_t d1,
                  uint64_t d2, uint64_t stride1_bytes, uint64_t stride2_bytes, uint32_t b0,
                  uint32_t b1, int swizzle) {
  cuuint64_t dims[3] = {d0, d1, d2};
  cuuint64_t strides[2] = {stride1_bytes, stride2_bytes};
  cuuint32_t box[3] = {b0, b1, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = d.tiled(m, tmap_dtype(t), 3, const_cast<void*>(ptr), dims, strides, box, estr,
                       CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle_enum(swizzle),
                       CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? HB_OK : HB_ERR_LAUNCH;
}

struct ConvGeom {
  int N, H, W, CI, CO, KH, KW, stride_h, stride_w, pad_h, pad_w, dil_h, dil_w, HO, WO;
  bool out_nchw;  // the conv kernel writes (N, CO, HO, WO)
  // byte strides of the input's W, H and N axes when it is not a dense NHWC tensor (0: dense)
  long long w_stride, h_stride, n_stride;
  int kslab;  // > 1: split-K into that many workspace slabs (see KParams::kslab)
  // 3-D convolution (see is_3d): depth extent, taps, stride, padding and output extent
  int D, KD, stride_d, pad_d, DO;
};

// (a padded depth axis of extent one still has more than one output plane)
bool is_3d(const ConvGeom& g) { return g.D > 1 || g.KD > 1 || g.pad_d > 0; }

}  // namespace

// A launch-ready kernel configuration: encoded tensor maps, kernel parameters, grid and shared
// memory size.  The counterpart of the module the reference gets back from tvm.build.
struct hb_plan {
  CUtensorMap tmA, tmB, tmC, tmB2;
  hb::KParams p;
  hb_knobs knobs;
  int grid;
  int smem;
  int owned_flags;  // hand-over flags (p.flags) this plan holds until it is destroyed; 0: none
  // what the output's tensor map was encoded from (TMA-store epilogue), for maps of further outputs
  int out_dt; long long out_d0, out_d1, out_d2;
  void* peer_maps_dev;  // device array of those maps (hb_plan_set_peer_outputs); freed with the plan
  // strip conv (conv_algo 2): its own parameter block; tmA = tiled input map, tmB = filter map
  bool strip;
  hb::StripParams sp;
  // wide strip conv (conv_algo 3): channels on the MMA's M axis, up to 256 pixels on N
  bool strip_t;
  hb::StripTParams spt;
  // NCHW operators only: one launch that brings input and filter to NHWC / HWIO first (the conv
  // kernel's epilogue writes NCHW itself)
  bool has_pre, pre_is_stem;
  hb::NchwPre pre;
  hb::StemPre stem;
  int pre_esize, pre_grid;
  // split-K NCHW plans: the kernel that sums the workspace slabs into the NCHW output
  bool has_post;
  const void* post_ws; void* post_out;
  int post_slabs, post_P, post_CO, post_N, post_kind;  // kind 0: float -> half, 1: float -> float, 2: int32
  long long post_slab_elems;
  // scan only: the kernel that writes the constant triangular operand first
  void* scan_b;
  int scan_N, scan_K, scan_es, scan_blocks;
  // packed-filter conv only: the unpack kernel that runs first on the same stream
  const void* packed_w;
  void* scratch;
  int unpack_blocks, sco, KH;
};

// ---- built-in scratch for callers that cannot allocate ---------------------------------------
// Device memory that lives inside the library image: every GPU that loads the library keeps
// these bytes until the process exits.  Host code must not use the array's name as a pointer
// (on the host it is only a handle for the runtime); set-up asks the runtime for the device
// address once per device and the kernels get that address as an ordinary argument.
#define HB_STATIC_SCRATCH_BYTES (4u << 20)
static __device__ __align__(256) int8_t g_hb_static_scratch[HB_STATIC_SCRATCH_BYTES];

// Hand-over flags (KParams::flags): one int per sliced tile of a split-K plan, or one per (CTA
// pair, epilogue warp) of a balanced plan; zero between launches.  A plan created with hb_plan_*
// owns its run of slots until hb_plan_destroy, so two live plans never share flags and may run
// on different streams at once; one plan must not run concurrently with itself.  The immediate
// entry points (hb_gemm, ...) take a run from a rotating cursor over the slots no live plan
// owns: two immediate calls whose kernels overlap on the GPU could share flags only after the
// cursor has gone round the whole array in between.
#define HB_FLAG_SLOTS 65536
static __device__ int g_hb_split_flags[HB_FLAG_SLOTS];

namespace {

constexpr int kMaxDevices = 64;
int* g_split_flags_addr[kMaxDevices] = {nullptr};
unsigned g_split_flags_cursor = 0;
void* g_static_scratch_addr[kMaxDevices] = {nullptr};
std::mutex g_static_scratch_mutex;

// Slots owned by live plans (process-wide: a plan's slots are reserved on every device).
unsigned char g_split_flags_owned[HB_FLAG_SLOTS] = {0};
// Set while hb_plan_* builds a heap plan: its flags are marked owned and freed on destroy.
thread_local bool g_plan_owns_flags = false;

// `count` consecutive flags of the current device's flag array (see g_hb_split_flags) that no
// live plan owns.  HB_ERR_SCRATCH when no such run is left (the caller then plans without them).
int split_flags(int count, int** out) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return HB_ERR_DEVICE;
  if (count <= 0 || count > HB_FLAG_SLOTS) return HB_ERR_SCRATCH;
  std::lock_guard<std::mutex> lock(g_static_scratch_mutex);
  if (g_split_flags_addr[dev] == nullptr) {
    void* ptr = nullptr;
    if (cudaGetSymbolAddress(&ptr, g_hb_split_flags) != cudaSuccess || ptr == nullptr) {
      cudaGetLastError();
      return HB_ERR_LAUNCH;
    }
    g_split_flags_addr[dev] = static_cast<int*>(ptr);
  }
  // next fit from the cursor, then once more from the start of the array
  const unsigned n = static_cast<unsigned>(count);
  auto find = [&](unsigned lo) -> long {
    unsigned at = lo;
    while (at + n <= HB_FLAG_SLOTS) {
      unsigned run = 0;
      while (run < n && !g_split_flags_owned[at + run]) ++run;
      if (run == n) return static_cast<long>(at);
      at += run + 1;  // past the owned slot that ended the run
    }
    return -1;
  };
  long found = find(g_split_flags_cursor);
  if (found < 0) found = find(0);
  if (found < 0) return HB_ERR_SCRATCH;
  const unsigned start = static_cast<unsigned>(found);
  if (g_plan_owns_flags)
    for (int i = 0; i < count; ++i) g_split_flags_owned[start + i] = 1;
  *out = g_split_flags_addr[dev] + start;
  g_split_flags_cursor = start + count;
  return HB_OK;
}

void release_split_flags(const int* flags, int count) {
  if (!flags || count <= 0) return;
  std::lock_guard<std::mutex> lock(g_static_scratch_mutex);
  for (int dev = 0; dev < kMaxDevices; ++dev) {
    const int* base = g_split_flags_addr[dev];
    if (base && flags >= base && flags + count <= base + HB_FLAG_SLOTS) {
      for (int i = 0; i < count; ++i) g_split_flags_owned[(flags - base) + i] = 0;
      return;
    }
  }
}

// Device address of g_hb_static_scratch on the current device (looked up on first use there).
int static_scratch_address(void** out) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return HB_ERR_DEVICE;
  std::lock_guard<std::mutex> lock(g_static_scratch_mutex);
  if (g_static_scratch_addr[dev] == nullptr) {
    void* ptr = nullptr;
    if (cudaGetSymbolAddress(&ptr, g_hb_static_scratch) != cudaSuccess || ptr == nullptr) {
      cudaGetLastError();  // leave no sticky error behind
      return HB_ERR_LAUNCH;
    }
    g_static_scratch_addr[dev] = ptr;
  }
  *out = g_static_scratch_addr[dev];
  return HB_OK;
}

}  // namespace
