// The C ABI of libheron_b200.so (include/heron_b200.h): every entry point checks its arguments,
// builds a plan (tensor maps, knobs, launch geometry) and enqueues it, or hands the plan back.
#include "hb_plan_conv.cuh"

extern "C" {

size_t hb_conv2d_nchw_scratch_bytes(int N, int H, int W, int CI, int CO, int KH, int KW,
                                    int stride_h, int stride_w, int pad, hb_dtype in_a,
                                    hb_dtype out_t) {
  NchwLayout L;
  return nchw_layout(N, H, W, CI, CO, KH, KW, stride_h, stride_w, pad, pad, in_a, out_t, &L) ? L.total : 0;
}

int hb_conv2d_nchw(const void* in, const void* w, void* out, int N, int H, int W, int CI, int CO,
                   int KH, int KW, int stride_h, int stride_w, int pad, hb_dtype in_a,
                   hb_dtype in_w, hb_dtype out_t, void* scratch, size_t scratch_bytes,
                   const hb_knobs* knobs, void* stream) {
  hb_plan plan;
  const int rc = plan_conv_nchw(in, w, out, N, H, W, CI, CO, KH, KW, stride_h, stride_w, pad, pad, in_a,
                                in_w, out_t, scratch, scratch_bytes, knobs, &plan);
  return rc != HB_OK ? rc : run_plan(&plan, static_cast<cudaStream_t>(stream));
}

int hb_plan_conv2d_nchw(hb_plan** plan, const void* in, const void* w, void* out, int N, int H,
                        int W, int CI, int CO, int KH, int KW, int stride_h, int stride_w, int pad,
                        hb_dtype in_a, hb_dtype in_w, hb_dtype out_t, void* scratch,
                        size_t scratch_bytes, const hb_knobs* knobs) {
  return new_plan(plan, [&](hb_plan* p) {
    return plan_conv_nchw(in, w, out, N, H, W, CI, CO, KH, KW, stride_h, stride_w, pad, pad, in_a, in_w,
                          out_t, scratch, scratch_bytes, knobs, p);
  });
}

int hb_version(void) { return 100; }

int hb_kernel_limits(hb_limits* out) {
  if (!out) return HB_ERR_SHAPE;
  out->max_shared_memory_per_block = kSmemLimit;
  out->tmem_columns = 512;
  out->tile_m = hb::kTileM;
  out->max_stages = hb::kMaxStages;
  out->epilogue_staging_bytes = hb::kUmmaEpiBytes;
  out->smem_slack_bytes = kSmemSlack;
  out->static_scratch_bytes = static_cast<int>(HB_STATIC_SCRATCH_BYTES);
  out->reserved = 0;
  return HB_OK;
}

int hb_sm_count(void) {
  Driver& d = driver();
  return d.status == HB_OK ? d.sm_count : -d.status;
}

int hb_default_knobs(int op, int batch, int M, int N, int K, int k_inner, hb_dtype in_a,
                     hb_dtype out, hb_knobs* k) {
  if (!k) return HB_ERR_KNOB;
  if (batch <= 0 || M <= 0 || N <= 0 || K <= 0 || k_inner <= 0) return HB_ERR_SHAPE;
  Problem pr{op, batch, M, N, K, in_a, in_a, out, op == 2, k_inner};
  resolve_knobs(pr, nullptr, 148, k);
  return HB_OK;
}

int hb_check_knobs(int op, int batch, int M, int N, int K, int k_inner, hb_dtype in_a,
                   hb_dtype out, const hb_knobs* k, int* smem_bytes, int* tmem_cols) {
  if (!k) return HB_ERR_KNOB;
  if (batch <= 0 || M <= 0 || N <= 0 || K <= 0 || k_inner <= 0) return HB_ERR_SHAPE;
  Problem pr{op, batch, M, N, K, in_a, in_a, out, op == 2, k_inner};
  hb_knobs full;
  resolve_knobs(pr, k, 148, &full);
  return check_knobs(pr, full, smem_bytes, tmem_cols);
}

int hb_balanced_run(int tiles, int stages_per_tile, int pairs, int pair, int* first, int* end) {
  if (tiles <= 0 || stages_per_tile <= 0 || pairs <= 0 || pair < 0 || pair >= pairs || !first || !end)
    return HB_ERR_SHAPE;
  const long long total = static_cast<long long>(tiles) * stages_per_tile;
  if (total > 0x7fffffffLL) return HB_ERR_SHAPE;
  *first = hb::sk_bound_of(static_cast<int>(total), stages_per_tile, kBalanceMinRun, pair, pairs);
  *end = hb::sk_bound_of(static_cast<int>(total), stages_per_tile, kBalanceMinRun, pair + 1, pairs);
  return HB_OK;
}

int hb_balanced_pieces(int tiles, int stages_per_tile, int pairs, int pair, int* pieces, int max_pieces) {
  if (tiles <= 0 || stages_per_tile <= 0 || pairs <= 0 || pair < 0 || pair >= pairs || !pieces || max_pieces < 0)
    return -HB_ERR_SHAPE;
  const long long total = static_cast<long long>(tiles) * stages_per_tile;
  if (total > 0x7fffffffLL) return -HB_ERR_SHAPE;
  hb::KParams p;
  std::memset(&p, 0, sizeof(p));
  p.sk = 1;
  p.sk_total = static_cast<int>(total);
  p.sk_per_tile = stages_per_tile;
  p.sk_min = kBalanceMinRun;
  hb::Walk w = hb::walk_begin(p, pair, pairs);
  hb::Piece pc;
  int n = 0;
  while (hb::walk_next(p, w, pc)) {
    if (n < max_pieces) {
      pieces[3 * n] = pc.t;
      pieces[3 * n + 1] = pc.s0;
      pieces[3 * n + 2] = pc.s1;
    }
    ++n;
  }
  return n;
}

int hb_gemm(const void* A, const void* B, void* C, int M, int K, int N, hb_dtype in_a,
            hb_dtype in_b, hb_dtype out, const hb_knobs* knobs, void* stream) {
  hb_plan plan;
  const int rc = plan_gemm_like(0, A, B, C, 1, M, K, N, in_a, in_b, out, knobs, &plan);
  return rc != HB_OK ? rc : run_plan(&plan, static_cast<cudaStream_t>(stream));
}

int hb_bmm(const void* A, const void* B, void* C, int batch, int M, int K, int N, hb_dtype in_a,
           hb_dtype in_b, hb_dtype out, const hb_knobs* knobs, void* stream) {
  hb_plan plan;
  const int rc = plan_gemm_like(1, A, B, C, batch, M, K, N, in_a, in_b, out, knobs, &plan);
  return rc != HB_OK ? rc : run_plan(&plan, static_cast<cudaStream_t>(stream));
}

// Matrix-vector product in the reference's tensor-core form: the vector is row 0 of an 8-row
// B whose other rows are zero, the result is column 0 of an (M, 8) output.  B's tensor map covers
// the one real row; TMA's out-of-bounds fill supplies the zero rows, so no padded copy is made.
int hb_gemv(const void* A, const void* x, void* out, int M, int K, hb_dtype in_a, hb_dtype in_x,
            hb_dtype out_t, const hb_knobs* knobs, void* stream) {
  hb_plan plan;
  const int rc = plan_gemm_like(0, A, x, out, 1, M, K, 8, in_a, in_x, out_t, knobs, &plan, 1);
  return rc != HB_OK ? rc : run_plan(&plan, static_cast<cudaStream_t>(stream));
}

int hb_plan_gemv(hb_plan** plan, const void* A, const void* x, void* out, int M, int K,
                 hb_dtype in_a, hb_dtype in_x, hb_dtype out_t, const hb_knobs* knobs) {
  return new_plan(plan, [&](hb_plan* p) {
    return plan_gemm_like(0, A, x, out, 1, M, K, 8, in_a, in_x, out_t, knobs, p, 1);
  });
}

// 3-D convolution, NCDHW: the NCHW machinery with a depth axis (5-D im2col loads in the kernel).
size_t hb_conv3d_ncdhw_scratch_bytes(int N, int D, int H, int W, int CI, int CO, int KD, int KH, int KW,
                                     int stride_d, int stride_h, int stride_w, int pad, hb_dtype in_a,
                                     hb_dtype out_t) {
  NchwLayout L;
  return nchw_layout(N, H, W, CI, CO, KH, KW, stride_h, stride_w, pad, pad, in_a, out_t, &L,
                     Depth{D, KD, stride_d, pad}) ? L.total : 0;
}

int hb_conv3d_ncdhw(const void* in, const void* w, void* out, int N, int D, int H, int W, int CI, int CO,
                    int KD, int KH, int KW, int stride_d, int stride_h, int stride_w, int pad,
                    hb_dtype in_a, hb_dtype in_w, hb_dtype out_t, void* scratch, size_t scratch_bytes,
                    const hb_knobs* knobs, void* stream) {
  hb_plan plan;
  const int rc = plan_conv_nchw(in, w, out, N, H, W, CI, CO, KH, KW, stride_h, stride_w, pad, pad, in_a, in_w,
                                out_t, scratch, scratch_bytes, knobs, &plan, Depth{D, KD, stride_d, pad});
  return rc != HB_OK ? rc : run_plan(&plan, static_cast<cudaStream_t>(stream));
}

int hb_plan_conv3d_ncdhw(hb_plan** plan, const void* in, const void* w, void* out, int N, int D, int H,
                         int W, int CI, int CO, int KD, int KH, int KW, int stride_d, int stride_h,
                         int stride_w, int pad, hb_dtype in_a, hb_dtype in_w, hb_dtype out_t,
                         void* scratch, size_t scratch_bytes, const hb_knobs* knobs) {
  return new_plan(plan, [&](hb_plan* p) {
    return plan_conv_nchw(in, w, out, N, H, W, CI, CO, KH, KW, stride_h, stride_w, pad, pad, in_a, in_w, out_t,
                          scratch, scratch_bytes, knobs, p, Depth{D, KD, stride_d, pad});
  });
}

size_t hb_scan_scratch_bytes(int N, int K, hb_dtype in_a) {
  if (N <= 0 || K <= 0) return 0;
  return static_cast<size_t>(N) * K * (in_a == HB_F16 ? 2 : 1);
}

int hb_scan(const void* A, void* out, int M, int N, int K, hb_dtype in_a, hb_dtype out_t, void* scratch,
            size_t scratch_bytes, const hb_knobs* knobs, void* stream) {
  hb_plan plan;
  const int rc = plan_scan(A, out, M, N, K, in_a, out_t, scratch, scratch_bytes, knobs, &plan);
  return rc != HB_OK ? rc : run_plan(&plan, static_cast<cudaStream_t>(stream));
}

int hb_plan_scan(hb_plan** plan, const void* A, void* out, int M, int N, int K, hb_dtype in_a,
                 hb_dtype out_t, void* scratch, size_t scratch_bytes, const hb_knobs* knobs) {
  return new_plan(plan, [&](hb_plan* p) {
    return plan_scan(A, out, M, N, K, in_a, out_t, scratch, scratch_bytes, knobs, p);
  });
}

// 1-D convolutions: the 2-D kernels with H = KH = 1 and no padding along the height.
size_t hb_conv1d_ncw_scratch_bytes(int N, int W, int CI, int CO, int KW, int stride, int pad,
                                   hb_dtype in_a, hb_dtype out_t) {
  NchwLayout L;
  return nchw_layout(N, 1, W, CI, CO, 1, KW, 1, stride, 0, pad, in_a, out_t, &L) ? L.total : 0;
}

int hb_conv1d_ncw(const void* in, const void* w, void* out, int N, int W, int CI, int CO, int KW,
                  int stride, int pad, hb_dtype in_a, hb_dtype in_w, hb_dtype out_t, void* scratch,
                  size_t scratch_bytes, const hb_knobs* knobs, void* stream) {
  hb_plan plan;
  const int rc = plan_conv_nchw(in, w, out, N, 1, W, CI, CO, 1, KW, 1, stride, 0, pad, in_a, in_w,
                                out_t, scratch, scratch_bytes, knobs, &plan);
  return rc != HB_OK ? rc : run_plan(&plan, static_cast<cudaStream_t>(stream));
}

int hb_plan_conv1d_ncw(hb_plan** plan, const void* in, const void* w, void* out, int N, int W,
                       int CI, int CO, int KW, int stride, int pad, hb_dtype in_a, hb_dtype in_w,
                       hb_dtype out_t, void* scratch, size_t scratch_bytes, const hb_knobs* knobs) {
  return new_plan(plan, [&](hb_plan* p) {
    return plan_conv_nchw(in, w, out, N, 1, W, CI, CO, 1, KW, 1, stride, 0, pad, in_a, in_w, out_t,
                          scratch, scratch_bytes, knobs, p);
  });
}

int hb_conv1d_nwc_packed(const void* in, const void* w_packed, void* out, int N, int W, int CI,
                         int CO, int KW, int stride, int pad, int dil, int sco, void* scratch,
                         size_t scratch_bytes, const hb_knobs* knobs, void* stream) {
  hb_plan plan;
  const int rc = plan_conv_packed(in, w_packed, out, N, 1, W, CI, CO, 1, KW, 1, stride, 0, pad, 1, dil,
                                  sco, scratch, scratch_bytes, knobs, &plan);
  return rc != HB_OK ? rc : run_plan(&plan, static_cast<cudaStream_t>(stream));
}

int hb_plan_conv1d_nwc_packed(hb_plan** plan, const void* in, const void* w_packed, void* out, int N,
                              int W, int CI, int CO, int KW, int stride, int pad, int dil, int sco,
                              void* scratch, size_t scratch_bytes, const hb_knobs* knobs) {
  return new_plan(plan, [&](hb_plan* p) {
    return plan_conv_packed(in, w_packed, out, N, 1, W, CI, CO, 1, KW, 1, stride, 0, pad, 1, dil, sco,
                            scratch, scratch_bytes, knobs, p);
  });
}

int hb_conv2d_nhwc(const void* in, const void* w, void* out, int N, int H, int W, int CI, int CO,
                   int KH, int KW, int stride_h, int stride_w, int pad, int dil_h, int dil_w,
                   hb_dtype in_a, hb_dtype in_w, hb_dtype out_t, const hb_knobs* knobs,
                   void* stream) {
  hb_plan plan;
  const int rc = plan_conv(in, w, out, N, H, W, CI, CO, KH, KW, stride_h, stride_w, pad, pad, dil_h,
                           dil_w, in_a, in_w, out_t, knobs, &plan);
  return rc != HB_OK ? rc : run_plan(&plan, static_cast<cudaStream_t>(stream));
}


size_t hb_conv2d_packed_scratch_bytes(int CI, int CO, int KH, int KW) {
  if (CI <= 0 || CO <= 0 || KH <= 0 || KW <= 0) return 0;
  return static_cast<size_t>(KH) * KW * CI * CO;
}

int hb_conv2d_nhwc_packed(const void* in, const void* w_packed, void* out, int N, int H, int W,
                          int CI, int CO, int KH, int KW, int stride_h, int stride_w, int pad,
                          int dil_h, int dil_w, int sco, void* scratch, size_t scratch_bytes,
                          const hb_knobs* knobs, void* stream) {
  hb_plan plan;
  const int rc = plan_conv_packed(in, w_packed, out, N, H, W, CI, CO, KH, KW, stride_h, stride_w,
                                  pad, pad, dil_h, dil_w, sco, scratch, scratch_bytes, knobs, &plan);
  return rc != HB_OK ? rc : run_plan(&plan, static_cast<cudaStream_t>(stream));
}

size_t hb_conv2d_packed_noalloc_max_bytes(void) { return HB_STATIC_SCRATCH_BYTES; }

int hb_conv2d_nhwc_packed_noalloc(const void* in, const void* w_packed, void* out, int N, int H,
                                  int W, int CI, int CO, int KH, int KW, int stride_h,
                                  int stride_w, int pad, int dil_h, int dil_w, int sco,
                                  const hb_knobs* knobs, void* stream) {
  const size_t need = hb_conv2d_packed_scratch_bytes(CI, CO, KH, KW);
  if (need == 0) return HB_ERR_SHAPE;
  if (need > HB_STATIC_SCRATCH_BYTES) return HB_ERR_STATIC_SCRATCH;
  Driver& d = driver();
  if (d.status != HB_OK) return d.status;
  void* scratch = nullptr;
  int rc = static_scratch_address(&scratch);
  if (rc != HB_OK) return rc;
  // The unpack kernel rewrites every byte of the scratch the conv kernel will read (the whole
  // KH*KW*CI*CO filter), so nothing left over from an earlier call can leak into this one.
  hb_plan plan;
  rc = plan_conv_packed(in, w_packed, out, N, H, W, CI, CO, KH, KW, stride_h, stride_w, pad, pad, dil_h,
                        dil_w, sco, scratch, HB_STATIC_SCRATCH_BYTES, knobs, &plan);
  return rc != HB_OK ? rc : run_plan(&plan, static_cast<cudaStream_t>(stream));
}

int hb_plan_gemm(hb_plan** plan, const void* A, const void* B, void* C, int M, int K, int N,
                 hb_dtype in_a, hb_dtype in_b, hb_dtype out, const hb_knobs* knobs) {
  return new_plan(plan, [&](hb_plan* p) {
    return plan_gemm_like(0, A, B, C, 1, M, K, N, in_a, in_b, out, knobs, p);
  });
}

int hb_plan_bmm(hb_plan** plan, const void* A, const void* B, void* C, int batch, int M, int K,
                int N, hb_dtype in_a, hb_dtype in_b, hb_dtype out, const hb_knobs* knobs) {
  return new_plan(plan, [&](hb_plan* p) {
    return plan_gemm_like(1, A, B, C, batch, M, K, N, in_a, in_b, out, knobs, p);
  });
}

int hb_plan_conv2d_nhwc(hb_plan** plan, const void* in, const void* w, void* out, int N, int H,
                        int W, int CI, int CO, int KH, int KW, int stride_h, int stride_w, int pad,
                        int dil_h, int dil_w, hb_dtype in_a, hb_dtype in_w, hb_dtype out_t,
                        const hb_knobs* knobs) {
  return new_plan(plan, [&](hb_plan* p) {
    return plan_conv(in, w, out, N, H, W, CI, CO, KH, KW, stride_h, stride_w, pad, pad, dil_h, dil_w,
                     in_a, in_w, out_t, knobs, p);
  });
}

int hb_plan_conv2d_nhwc_packed(hb_plan** plan, const void* in, const void* w_packed, void* out,
                               int N, int H, int W, int CI, int CO, int KH, int KW, int stride_h,
                               int stride_w, int pad, int dil_h, int dil_w, int sco, void* scratch,
                               size_t scratch_bytes, const hb_knobs* knobs) {
  return new_plan(plan, [&](hb_plan* p) {
    return plan_conv_packed(in, w_packed, out, N, H, W, CI, CO, KH, KW, stride_h, stride_w, pad, pad,
                            dil_h, dil_w, sco, scratch, scratch_bytes, knobs, p);
  });
}

int hb_plan_launch(const hb_plan* plan, void* stream) {
  if (!plan) return HB_ERR_SHAPE;
  return run_plan(plan, static_cast<cudaStream_t>(stream));
}

int hb_plan_knobs(const hb_plan* plan, hb_knobs* knobs, int* grid, int* smem_bytes) {
  if (!plan || !knobs) return HB_ERR_SHAPE;
  *knobs = plan->knobs;
  if (grid) *grid = plan->grid;
  if (smem_bytes) *smem_bytes = plan->smem;
  return HB_OK;
}

int hb_plan_set_peer_outputs(hb_plan* plan, int n, void* const* outs) { return set_peer_outputs(plan, n, outs); }

void hb_plan_destroy(hb_plan* plan) { destroy_plan(plan); }

int hb_last_status(int* status) {
  if (!status) return HB_ERR_SHAPE;
  Driver& d = driver();
  if (d.status != HB_OK) return d.status;
  if (cudaDeviceSynchronize() != cudaSuccess) return HB_ERR_LAUNCH;
  int v = 0;
  if (cudaMemcpyFromSymbol(&v, hb::g_hb_status, sizeof(int)) != cudaSuccess) return HB_ERR_LAUNCH;
  *status = v;
  if (v != 0) {
    const int zero = 0;
    if (cudaMemcpyToSymbol(hb::g_hb_status, &zero, sizeof(int)) != cudaSuccess) return HB_ERR_LAUNCH;
    // a kernel that gave up may have left turn-taking flags of its split-K tiles half way
    void* flags = nullptr;
    if (cudaGetSymbolAddress(&flags, g_hb_split_flags) == cudaSuccess && flags)
      cudaMemset(flags, 0, sizeof(int) * HB_FLAG_SLOTS);
  }
  return HB_OK;
}

const char* hb_status_string(int status) {
  switch (status) {
    case HB_OK: return "ok";
    case HB_ERR_SHAPE: return "shape outside the kernel's documented limits";
    case HB_ERR_ALIGN: return "null or misaligned pointer (16-byte alignment required)";
    case HB_ERR_KNOB: return "knob set outside the constrained space";
    case HB_ERR_LAUNCH: return "CUDA launch or tensor-map encoding failed";
    case HB_ERR_TIMEOUT: return "a bounded device-side wait ran out";
    case HB_ERR_DEVICE: return "no usable sm_100 device";
    case HB_ERR_DTYPE: return "unsupported dtype combination";
    case HB_ERR_SCRATCH: return "scratch buffer missing or too small";
    case HB_ERR_STATIC_SCRATCH:
      return "filter does not fit the library's built-in 4 MiB scratch (hb_conv2d_nhwc_packed_noalloc)";
  }
  return "unknown status";
}

}  // extern "C"
