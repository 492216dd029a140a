/*
 * heron_b200.h — C ABI of libheron_b200.so.
 *
 * The library holds hand-written sm_100a kernels (tcgen05 MMA, TMEM accumulators, TMA-fed
 * shared-memory ring) for the tensor programs that the Heron auto-tuner generates through TVM:
 * GEMM, batched GEMM and NHWC conv2d, in fp16 -> fp32/fp16 and u8/s8 -> s32.
 *
 * What each entry point replaces in the reference: the TVM-built packed function that
 * Task.instantiate() hands to tvm.build (task/task.py:76-89).  Its arguments are the operator's
 * input tensors followed by its output tensor (task/task.py:81), all allocated by the caller
 * (tests/quick_start/dlboost/run.py:52-58); the callee allocates and frees nothing.  The entry
 * points below keep that contract: plain device pointers and sizes, caller-owned buffers, a CUDA
 * stream, and an int status in place of a TVMError (runner/measure_methods.py:178-185).
 *
 * There is no CPU fallback anywhere in this library: without a Blackwell GPU every compute entry
 * point returns HB_ERR_DEVICE.
 */
#ifndef HERON_B200_H_
#define HERON_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- status codes ------------------------------------------------------------------------ */
enum {
  HB_OK = 0,
  HB_ERR_SHAPE = 1,   /* a dimension is non-positive or breaks a documented divisibility rule   */
  HB_ERR_ALIGN = 2,   /* a pointer is not 16-byte aligned, or a row pitch is not a 16-byte multiple */
  HB_ERR_KNOB = 3,    /* the knob set is outside the kernel's constrained space                  */
  HB_ERR_LAUNCH = 4,  /* the CUDA runtime or driver refused the launch / tensor-map encoding    */
  HB_ERR_TIMEOUT = 5, /* a bounded device-side wait ran out; read by hb_last_status            */
  HB_ERR_DEVICE = 6,  /* no usable sm_100 device                                                 */
  HB_ERR_DTYPE = 7,   /* dtype combination the kernels do not implement                         */
  HB_ERR_SCRATCH = 8, /* the caller's scratch buffer is missing or too small                    */
  HB_ERR_STATIC_SCRATCH = 9 /* the problem needs more than the library's built-in scratch array */
};

/* ---- element types ----------------------------------------------------------------------- */
typedef enum {
  HB_F16 = 0, /* IEEE binary16 */
  HB_F32 = 1,
  HB_S8 = 2,
  HB_U8 = 3,
  HB_S32 = 4
} hb_dtype;

/*
 * Knobs of the kernel family: the tile / stage / raster parameters a tuner may choose.  They
 * take the place of the reference's wmma fragment and tiling knobs
 * (schedule/sched_op/gpu_tensorcore_operator.py:282-294, schedule/sched_op/sched_common.py:157-170).
 * A zero in any field means "library default for this shape".
 */
typedef struct {
  int tile_n;        /* accumulator tile width; multiple of 32 (64 for fp16 output), 32..256      */
  int stages;        /* depth of the TMA -> MMA shared-memory ring, 1..12                          */
  int swizzle_bytes; /* bytes of K per ring stage and TMA swizzle span: 32, 64 or 128             */
  int acc_stages;    /* TMEM accumulator buffers (1 or 2); 2 overlaps epilogue with the next tile */
  int raster;        /* 0: consecutive tiles walk N first (default); 1: walk M first               */
  int epilogue;      /* 1: TMEM -> registers -> shared memory -> TMA store; 2: direct global stores */
  int max_ctas;      /* cap on the persistent grid (0: one CTA per SM)                             */
  int cta_group;     /* 1: each CTA owns its MMAs (128 x tile_n tiles); 2: CTA pairs share them
                        (tcgen05 cta_group::2, 256 x tile_n tiles, half of B staged per CTA)        */
  int l2_prefetch;   /* ring stages ahead of the loads at which operand tiles are prefetched into
                        L2; 0 = library default, -1 = off (gemm / bmm only)                         */
  int conv_algo;     /* conv only.  1: implicit GEMM, one im2col TMA per filter tap; 2: resident
                        filter + one padded input strip per tile (stride 1, filter fits shared
                        memory, padded width <= 128); 3: the same with the operands' places changed:
                        output channels on the MMA's M axis (64 or 128 of them), 256 consecutive
                        output positions on N (fp16, stride 1; tile_n then caps the positions per
                        tile, rounded down to a multiple of 64); 4: algorithm 2 with the three taps
                        of a filter row taken by one MMA of 192 columns, the epilogue adding the
                        column groups shifted by one and two pixels (fp16, 64 output channels,
                        KW = 3, no dilation along W); 0 = library picks                            */
  int tail_split;    /* the tiles of the last, partly filled wave of the persistent grid are cut into
                        this many column slices (1, 2 or 4); 0 = library picks                      */
  int split_k;       /* work items that do not fill a wave of the persistent grid (the tiles of the
                        last wave, or all tiles of a small problem) are cut into this many slices of
                        the reduction instead; the slices of a tile take turns: the first stores,
                        the next ones add (TMA reduce-add or red.global) once the one before has
                        finished, so the order of the additions is fixed.  1 = off, 2..4,
                        0 = library picks.  4-byte outputs only                                   */
  int k_slices;      /* swizzle spans of K behind one ring barrier (1 or 2): with 2 the MMA thread
                        waits, fences and commits once per eight MMAs instead of four, at the same
                        ring size in bytes.  0 = library picks                                     */
  int balance;       /* work distribution over the persistent CTAs (or CTA pairs).  1: whole tiles dealt
                        out round-robin (with tail_split / split_k for the last wave); 2: the (tile,
                        K stage) units of the whole problem in equal runs, one per CTA pair: tiles at
                        the ends of a run are shared with the neighbouring pair, which leaves its
                        partial sums in the output for this one to add (fixed order, no atomics;
                        overrides tail_split and split_k).  4-byte outputs with 16-byte rows only;
                        0 = library picks                                                          */
  int epi_warps;     /* warps that drain a CTA's accumulators: 4 (one per 32 TMEM lanes, two staging
                        buffers each) or 8 (two per 32 lanes, each with half of a tile's column
                        chunks and one staging buffer); 0 = library picks (8 where a tile's K loop
                        is shorter than its drain)                                                */
  int silent_producer; /* test hook, leave 0.  1: the TMA producers issue nothing, so every consumer's
                        bounded wait runs out (0.1 s limit for such a launch) and the launch ends
                        with HB_ERR_TIMEOUT in the status word and the context intact              */
  int probe;         /* diagnostic modes of builds made with -DHB_PROBES; ignored otherwise         */
} hb_knobs;

/*
 * The SM limits the kernels' knob space is built from, so that a host-side constraint model
 * (the reference registers thread and shared-memory limits the same way,
 * schedule/context/cuda_context.py:25-63) states the same bounds as hb_check_knobs.
 */
typedef struct {
  int max_shared_memory_per_block; /* opt-in dynamic shared memory per CTA, bytes              */
  int tmem_columns;                /* 32-bit accumulator columns per SM                         */
  int tile_m;                      /* rows of one CTA's accumulator tile                        */
  int max_stages;                  /* deepest TMA -> MMA ring                                   */
  int epilogue_staging_bytes;      /* shared memory the TMA-store epilogue takes                */
  int smem_slack_bytes;            /* alignment padding + barriers                              */
  int static_scratch_bytes;        /* capacity of the built-in scratch of the no-alloc entry    */
  int reserved;
} hb_limits;
int hb_kernel_limits(hb_limits* out);

/* Library / device facts. */
int hb_version(void);
/* Number of SMs of the current device, or a negative status. */
int hb_sm_count(void);
/* Fills *k with the defaults the library would pick for op (0 gemm, 1 bmm, 2 conv) on a problem
 * whose GEMM view is (batch, M, N, K) with the given dtypes.  k_inner is the contiguous part of
 * the reduction: K for gemm/bmm, the input channel count CI for conv. */
int hb_default_knobs(int op, int batch, int M, int N, int K, int k_inner, hb_dtype in_a,
                     hb_dtype out, hb_knobs* k);
/* Checks a knob set against the kernel's own limits (shared memory, TMEM columns, divisibility)
 * without touching the GPU.  Returns HB_OK or HB_ERR_KNOB; *smem_bytes / *tmem_cols receive the
 * resources the configuration needs (either may be NULL). */
int hb_check_knobs(int op, int batch, int M, int N, int K, int k_inner, hb_dtype in_a,
                   hb_dtype out, const hb_knobs* k, int* smem_bytes, int* tmem_cols);

/*
 * The partition rule of the balanced schedule (knob `balance` = 2), evaluated on the host: the
 * problem's `tiles` x `stages_per_tile` ring stages, numbered tile-major, are cut into `pairs`
 * runs; *first / *end receive the run [first, end) of CTA pair `pair`.  A cut that falls within
 * two stages of a tile edge is moved onto it.  It is the same function the kernel evaluates; a
 * tuner's cost model or a test can call it without a GPU.  The reference has no counterpart: its
 * generated kernels bind one block per output tile (schedule/sched_op/gpu_tensorcore_operator.py).
 */
int hb_balanced_run(int tiles, int stages_per_tile, int pairs, int pair, int* first, int* end);
/* The pieces of that run in the order the kernel's roles take them (the kernel's own walker,
 * compiled for the host): up to max_pieces triples (tile, first stage, end stage) are written to
 * `pieces`; returns the number of pieces of the run, or a negative status. */
int hb_balanced_pieces(int tiles, int stages_per_tile, int pairs, int pair, int* pieces, int max_pieces);

/*
 * GEMM: C[M,N] = sum_k A[M,K] * B[N,K]  (B is stored N-major over K, i.e. C = A * B^T).
 * Replaces the artefact built from ops/cuda/dense.py:4-17 (fp16 inputs; `in_b == in_a`) and
 * ops/x86/dense.py:6-18 (A uint8, B int8, C int32).  Accepted combinations:
 *   in_a = in_b = HB_F16, out = HB_F32 or HB_F16 (fp32 accumulation, RN conversion for HB_F16);
 *   in_a in {HB_U8, HB_S8}, in_b in {HB_U8, HB_S8}, out = HB_S32 (exact).
 * All three are dense row-major device buffers.  K*sizeof(in) must be a multiple of 16.
 */
int hb_gemm(const void* A, const void* B, void* C, int M, int K, int N, hb_dtype in_a,
            hb_dtype in_b, hb_dtype out, const hb_knobs* knobs, void* stream);

/*
 * Batched GEMM: C[b,M,N] = sum_k A[b,M,K] * B[b,N,K].  Replaces ops/cuda/batch_matmul.py:5-19 and
 * ops/x86/batch_matmul.py:6-20.  Same dtype table as hb_gemm.  batch >= 1 here (the reference op
 * asserts batch > 1 at ops/cuda/batch_matmul.py:6; the Python operator keeps that assert).
 */
int hb_bmm(const void* A, const void* B, void* C, int batch, int M, int K, int N, hb_dtype in_a,
           hb_dtype in_b, hb_dtype out, const hb_knobs* knobs, void* stream);

/*
 * NHWC conv2d as implicit GEMM:
 *   out[n,y,x,f] = sum_{ry,rx,rc} pad(in)[n, y*sh + ry*dh, x*sw + rx*dw, rc] * w[ry,rx,rc,f]
 * with `in` (N,H,W,CI), `w` HWIO (KH,KW,CI,CO) and `out` (N,HO,WO,CO), zero padding `pad` on all
 * four sides.  Replaces ops/cuda/conv2d.py:137-196; with in_a = HB_U8, in_w = HB_S8 it computes
 * what ops/x86/conv2d_int8.py:31-93 computes once that op's packed filter is unpacked to HWIO
 * (see hb_conv2d_nhwc_packed).  CI*sizeof(in) must be a multiple of 32 and CO*sizeof(out) of 16.
 */
int hb_conv2d_nhwc(const void* in, const void* w, void* out, int N, int H, int W, int CI, int CO,
                   int KH, int KW, int stride_h, int stride_w, int pad, int dil_h, int dil_w,
                   hb_dtype in_a, hb_dtype in_w, hb_dtype out_t, const hb_knobs* knobs,
                   void* stream);

/*
 * The x86 operator's own filter format (ops/x86/conv2d_int8.py:36-50): `w_packed` is int8 with
 * shape (CO/sco, KH, KW, CI/4, sco, 4), sco in {64, 48, 32} ("OhwI64o4i", "OhwI48o4i",
 * "OhwI32o4i"); input uint8 NHWC, output int32 (N,HO,WO,CO/sco,sco), which is NHWC.  The filter
 * is unpacked to HWIO into `scratch` (caller-owned device memory of at least
 * hb_conv2d_packed_scratch_bytes(...) bytes) by a small kernel on the same stream, then the
 * implicit-GEMM kernel runs on it.
 */
size_t hb_conv2d_packed_scratch_bytes(int CI, int CO, int KH, int KW);
int hb_conv2d_nhwc_packed(const void* in, const void* w_packed, void* out, int N, int H, int W,
                          int CI, int CO, int KH, int KW, int stride_h, int stride_w, int pad,
                          int dil_h, int dil_w, int sco, void* scratch, size_t scratch_bytes,
                          const hb_knobs* knobs, void* stream);

/*
 * NCHW conv2d, the operator the reference's network tables use
 * (ops/cuda/conv2d.py:9-135; tests/figure10/configs/resnet50.json):
 *   out[n,c,p,q] = sum_{ci,kh,kw} pad(in)[n, ci, p*sh+kh, q*sw+kw] * w[c,ci,kh,kw]
 * `in` (N,CI,H,W), `w` (CO,CI,KH,KW), `out` (N,CO,HO,WO), dilation 1 (the reference asserts it).
 * The reference lowers it to an explicit im2col GEMM; here one launch brings input and filter
 * to NHWC / HWIO in `scratch` (channels zero-padded to a 32-byte multiple, which also covers the
 * reference's CI == 3 special case: its zero-padded filter taps add nothing) and the conv
 * kernel's epilogue writes NCHW directly (for one channel a warp's 32 accumulator rows are 32
 * consecutive pixels).  `scratch` is caller-owned device memory, 256-byte aligned, of at least
 * hb_conv2d_nchw_scratch_bytes(...) bytes (the transposed input and filter).
 */
size_t hb_conv2d_nchw_scratch_bytes(int N, int H, int W, int CI, int CO, int KH, int KW,
                                    int stride_h, int stride_w, int pad, hb_dtype in_a,
                                    hb_dtype out_t);
int hb_conv2d_nchw(const void* in, const void* w, void* out, int N, int H, int W, int CI, int CO,
                   int KH, int KW, int stride_h, int stride_w, int pad, hb_dtype in_a,
                   hb_dtype in_w, hb_dtype out_t, void* scratch, size_t scratch_bytes,
                   const hb_knobs* knobs, void* stream);

/*
 * Operators next to the hot path that run on the same kernels.
 *
 * hb_gemv: the tensor-core matrix-vector product of ops/cuda/gemv.py:4-30.  `A` (M,K), `x` (1,K),
 * `out` (M,8): out[i,0] = sum_k A[i,k] * x[0,k], out[i,1..7] = 0 (the reference pads the vector to
 * an 8-row matrix of zeros so that a wmma fragment fits; the zeros are written here too, so the
 * buffer holds what the reference's would).  The x86 form (ops/x86/gemv.py:6-19: A (1,K), B (M,K),
 * out (1,M)) is hb_gemm with M = 1.
 *
 * hb_conv1d_ncw: ops/cuda/conv1d.py:11-110.  `in` (N,CI,W), `w` (CO,CI,KW), `out` (N,CO,WO),
 * WO = (W - KW + 2*pad) / stride + 1, dilation 1 (asserted there).  Runs as hb_conv2d_nchw with
 * H = KH = 1 and no padding along the height; `scratch` as for hb_conv2d_nchw, sized by
 * hb_conv1d_ncw_scratch_bytes.
 *
 * hb_conv1d_nwc_packed: ops/x86/conv1d_int8.py:31-101.  `in` uint8 (N,W,CI), `w_packed` int8
 * (CO/sco, KW, CI/4, sco, 4), `out` int32 (N, WO, CO/sco, sco), WO from the dilated kernel size.
 * Runs as hb_conv2d_nhwc_packed with H = KH = 1; scratch of hb_conv2d_packed_scratch_bytes(CI, CO,
 * 1, KW) bytes.
 *
 * hb_scan: ops/cuda/scan.py:4-23 and ops/x86/scan.py:6-27.  out[m,n] = sum_k A[m,k] * B[n,k] with
 * the constant B[n,k] = (n <= k) ? 0 : 1, i.e. out[m,n] = sum of A[m,k] over k < min(n, K): an
 * exclusive running sum written as a GEMM.  `A` (M,K) fp16, or uint8 for the x86 form (B is then
 * int8); `out` (M,N).  A kernel of the plan writes B into `scratch`
 * (hb_scan_scratch_bytes(N, K, in_a) bytes, 16-byte aligned) before the GEMM kernel reads it.
 */
int hb_gemv(const void* A, const void* x, void* out, int M, int K, hb_dtype in_a, hb_dtype in_x,
            hb_dtype out_t, const hb_knobs* knobs, void* stream);
size_t hb_scan_scratch_bytes(int N, int K, hb_dtype in_a);

/*
 * hb_conv3d_ncdhw: ops/cuda/conv3d.py:9-110.  `in` (N,CI,D,H,W), `w` (CO,CI,KD,KH,KW), `out`
 * (N,CO,DO,HO,WO); `pad` zeros on every side of the three spatial axes (an int padding in
 * get_pad_tuple3d), dilation 1 (asserted there):
 *   out[n,c,d,p,q] = sum_{ci,kd,kh,kw} pad(in)[n, ci, d*sd+kd, p*sh+kh, q*sw+kw] * w[c,ci,kd,kh,kw]
 * The glue of hb_conv2d_nchw brings input and filter to NDHWC / (KD,KH,KW,CI,CO); the conv kernel
 * reads the activations with 5-D im2col TMA loads (three tap offsets) and writes NCDHW.
 */
size_t hb_conv3d_ncdhw_scratch_bytes(int N, int D, int H, int W, int CI, int CO, int KD, int KH, int KW,
                                     int stride_d, int stride_h, int stride_w, int pad, hb_dtype in_a,
                                     hb_dtype out_t);
int hb_conv3d_ncdhw(const void* in, const void* w, void* out, int N, int D, int H, int W, int CI, int CO,
                    int KD, int KH, int KW, int stride_d, int stride_h, int stride_w, int pad,
                    hb_dtype in_a, hb_dtype in_w, hb_dtype out_t, void* scratch, size_t scratch_bytes,
                    const hb_knobs* knobs, void* stream);
int hb_scan(const void* A, void* out, int M, int N, int K, hb_dtype in_a, hb_dtype out_t, void* scratch,
            size_t scratch_bytes, const hb_knobs* knobs, void* stream);
size_t hb_conv1d_ncw_scratch_bytes(int N, int W, int CI, int CO, int KW, int stride, int pad,
                                   hb_dtype in_a, hb_dtype out_t);
int hb_conv1d_ncw(const void* in, const void* w, void* out, int N, int W, int CI, int CO, int KW,
                  int stride, int pad, hb_dtype in_a, hb_dtype in_w, hb_dtype out_t, void* scratch,
                  size_t scratch_bytes, const hb_knobs* knobs, void* stream);
int hb_conv1d_nwc_packed(const void* in, const void* w_packed, void* out, int N, int W, int CI,
                         int CO, int KW, int stride, int pad, int dil, int sco, void* scratch,
                         size_t scratch_bytes, const hb_knobs* knobs, void* stream);

/*
 * hb_conv2d_nhwc_packed without a scratch argument and without any allocation.  It has no
 * counterpart in the reference: it exists because the reference's calling convention has no room
 * for a workspace.  A built operator there receives exactly its tensors (input, filter, output;
 * task/task.py:81) and nothing else, so a host that drives this library through that convention
 * has no pointer to hand over, and it cannot call cudaMalloc either when the call sits inside a
 * timed measurement loop (cudaMalloc synchronises the device and would be measured) or inside a
 * region where allocation is forbidden outright, such as a stream capture or a serving loop with
 * a fixed memory budget.
 *
 * The unpacked filter goes into an array that is part of the library image
 * (hb_conv2d_packed_noalloc_max_bytes() = 4 MiB; every GPU that loads the library holds those
 * 4 MiB until the process exits).  A filter with KH*KW*CI*CO bytes above that limit is refused
 * with HB_ERR_STATIC_SCRATCH; use hb_conv2d_nhwc_packed with your own buffer instead.
 *
 * The first call on each device looks up the array's device address (cudaGetSymbolAddress);
 * make that first call outside any stream capture.  All calls on a device share the one array,
 * which keeps the last call's unpacked filter: every call rewrites all the bytes it later reads,
 * so nothing needs clearing, but two calls whose kernels can overlap on the GPU (different
 * streams, no dependency between them) race on it.  Calls on one stream are safe.
 * The entry point calls no cudaMalloc / cudaFree and no library routine that allocates.
 */
size_t hb_conv2d_packed_noalloc_max_bytes(void);
int hb_conv2d_nhwc_packed_noalloc(const void* in, const void* w_packed, void* out, int N, int H,
                                  int W, int CI, int CO, int KH, int KW, int stride_h,
                                  int stride_w, int pad, int dil_h, int dil_w, int sco,
                                  const hb_knobs* knobs, void* stream);

/*
 * Plans.  A plan is what the reference gets back from tvm.build on an instantiated schedule
 * (tests/quick_start/dlboost/run.py:44-46) and then calls many times under time_evaluator
 * (run.py:60-62): the encoded TMA tensor maps, the resolved knobs and the launch geometry for one
 * problem on fixed buffers.  Creating one costs three tensor-map encodings on the host and no
 * device work; hb_plan_launch only enqueues the kernel(s) and may be captured in a CUDA graph.
 * The argument lists are those of the immediate entry points above minus the stream.
 */
typedef struct hb_plan hb_plan;
int hb_plan_gemm(hb_plan** plan, const void* A, const void* B, void* C, int M, int K, int N,
                 hb_dtype in_a, hb_dtype in_b, hb_dtype out, const hb_knobs* knobs);
int hb_plan_bmm(hb_plan** plan, const void* A, const void* B, void* C, int batch, int M, int K,
                int N, hb_dtype in_a, hb_dtype in_b, hb_dtype out, const hb_knobs* knobs);
int hb_plan_conv2d_nhwc(hb_plan** plan, const void* in, const void* w, void* out, int N, int H,
                        int W, int CI, int CO, int KH, int KW, int stride_h, int stride_w, int pad,
                        int dil_h, int dil_w, hb_dtype in_a, hb_dtype in_w, hb_dtype out_t,
                        const hb_knobs* knobs);
int hb_plan_conv2d_nhwc_packed(hb_plan** plan, const void* in, const void* w_packed, void* out,
                               int N, int H, int W, int CI, int CO, int KH, int KW, int stride_h,
                               int stride_w, int pad, int dil_h, int dil_w, int sco, void* scratch,
                               size_t scratch_bytes, const hb_knobs* knobs);
int hb_plan_conv2d_nchw(hb_plan** plan, const void* in, const void* w, void* out, int N, int H,
                        int W, int CI, int CO, int KH, int KW, int stride_h, int stride_w, int pad,
                        hb_dtype in_a, hb_dtype in_w, hb_dtype out_t, void* scratch,
                        size_t scratch_bytes, const hb_knobs* knobs);
int hb_plan_conv3d_ncdhw(hb_plan** plan, const void* in, const void* w, void* out, int N, int D, int H,
                         int W, int CI, int CO, int KD, int KH, int KW, int stride_d, int stride_h,
                         int stride_w, int pad, hb_dtype in_a, hb_dtype in_w, hb_dtype out_t,
                         void* scratch, size_t scratch_bytes, const hb_knobs* knobs);
int hb_plan_scan(hb_plan** plan, const void* A, void* out, int M, int N, int K, hb_dtype in_a,
                 hb_dtype out_t, void* scratch, size_t scratch_bytes, const hb_knobs* knobs);
int hb_plan_gemv(hb_plan** plan, const void* A, const void* x, void* out, int M, int K,
                 hb_dtype in_a, hb_dtype in_x, hb_dtype out_t, const hb_knobs* knobs);
int hb_plan_conv1d_ncw(hb_plan** plan, const void* in, const void* w, void* out, int N, int W,
                       int CI, int CO, int KW, int stride, int pad, hb_dtype in_a, hb_dtype in_w,
                       hb_dtype out_t, void* scratch, size_t scratch_bytes, const hb_knobs* knobs);
int hb_plan_conv1d_nwc_packed(hb_plan** plan, const void* in, const void* w_packed, void* out, int N,
                              int W, int CI, int CO, int KW, int stride, int pad, int dil, int sco,
                              void* scratch, size_t scratch_bytes, const hb_knobs* knobs);
int hb_plan_launch(const hb_plan* plan, void* stream);
/* The knobs after defaults were resolved, the persistent grid and the dynamic shared memory. */
int hb_plan_knobs(const hb_plan* plan, hb_knobs* knobs, int* grid, int* smem_bytes);
/*
 * Further outputs of a gemm / bmm / conv2d_nhwc plan whose epilogue is the TMA store (`epilogue` 1,
 * no split-K, not the balanced schedule, not a strip kernel): every tile the kernel stores to the
 * plan's output is stored to each of `outs[0..n)` as well, straight from the same shared-memory
 * staging buffer.  Meant for the sharded operators (batches / images over the GPUs of one box,
 * heron_b200/multi.py): `outs` are this rank's slice of the other GPUs' full-size output buffers,
 * mapped into this process (CUDA IPC or symmetric memory), so the whole output is complete on
 * every GPU when every rank's kernel has finished and no collective runs afterwards.  The caller
 * orders "every rank has finished" itself (a barrier on the stream).  Each pointer 16-byte
 * aligned, same shape and layout as the plan's output; n <= 15; n = 0 removes them.  Allocates a
 * small device array for the tensor maps (freed by hb_plan_destroy).
 */
int hb_plan_set_peer_outputs(hb_plan* plan, int n, void* const* outs);
void hb_plan_destroy(hb_plan* plan);

/*
 * Device-side status of the kernels launched so far on the current device: synchronises the
 * device, copies the status word (HB_OK or HB_ERR_TIMEOUT) to *status and clears it.  A bounded
 * wait that ran out leaves the output undefined but the context usable.  Stands in for the
 * per-candidate error the reference's runner records (runner/measure_methods.py:178-185).
 */
int hb_last_status(int* status);

/* Human-readable text for a status code (static storage). */
const char* hb_status_string(int status);

#ifdef __cplusplus
}
#endif
#endif /* HERON_B200_H_ */
