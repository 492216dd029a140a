// The one kernel body behind GEMM, batched GEMM and NHWC conv2d (implicit GEMM).
//
//   D[b, m, n] = sum_k A[b, m, k] * B[b, n, k]
//
// Persistent CTAs (one per SM) walk a static list of 128 x BN output tiles.  Inside a CTA the
// warps have fixed roles:
//   warp 0      one elected lane issues the A-operand TMA loads into a ring of shared-memory
//               stages (and arms each stage's barrier with the bytes both operands will bring);
//   last warp   one elected lane issues the B-operand loads of the same stages (two issuing
//               threads keep more loads in flight than one: +12 % on the int8 conv);
//   warp 1      allocates TMEM; one elected lane issues tcgen05.mma into a TMEM accumulator and
//               commits stage-free / accumulator-full events to mbarriers;
//   warps 2..   epilogue, four or eight warps (chosen per launch): tcgen05.ld the accumulator
//               (a warp may touch the 32 TMEM lanes of its position in its warpgroup; with eight
//               warps the two of a position split a tile's 128-byte column chunks), convert, and
//               write the tile either through swizzled shared memory + TMA store or with direct
//               vector stores.  Eight pay where a tile's K loop is shorter than its drain.
// Two accumulator buffers in TMEM let the MMA warp start the next tile while the epilogue warps
// drain the previous one.
//
// A ring stage holds KS (1 or 2) swizzle spans of K per operand behind one "full" / "empty"
// barrier pair: with two, the MMA thread waits, fences and commits once per eight MMAs instead of
// four and the producers arm half as many barriers, at the same ring size in bytes.
//
// With CG = 2 the two CTAs of a cluster share every MMA (tcgen05 cta_group::2): the pair owns a
// 256 x BN tile, each CTA stages its own 128 rows of A and its own half of B's BN rows, the
// leader CTA (cluster rank 0) issues the instruction for both and each CTA's TMEM receives its
// 128 x BN half of the accumulator.  A CTA then pulls a third less operand data per flop than
// alone, which is what the large tensor-bound shapes are limited by.  Loads of both CTAs
// complete on the leader's "full" barrier; the leader's commits arrive on both CTAs' "empty"
// and "accumulator full" barriers; both CTAs' epilogue warps arrive on the leader's
// "accumulator empty" barrier.
//
// Operand layouts in shared memory are the canonical swizzled UMMA layouts, written by TMA:
//   A, K-major:   rows = M index, each row SW bytes of K (SW = 32/64/128 = TMA swizzle span);
//   B, K-major:   rows = N index, same (GEMM / BMM: B is stored (N, K));
//   B, MN-major:  rows = K index, each row SW bytes of N; BN*esize/SW such column chunks
//                 (conv: the HWIO filter is a (KH*KW*CI, CO) matrix with CO contiguous).
// For conv the A tile is fetched with im2col-mode TMA: 128 consecutive output pixels of one
// filter tap and one channel chunk, zero-filled where the tap falls into the padding.
//
// Work items are whole tiles, or — for the tiles that would leave a wave of the persistent grid
// partly empty — column slices of a tile or slices of its K range.  K slices either add into a
// zeroed output (TMA reduce-add / red.global) or are stored side by side into workspace slabs that
// a later kernel sums in a fixed order.  Other variants of the same body: A shared by all batches
// with B read as (K, N) tiles (a 1x1 NCHW conv on the tensors in place), a third spatial axis
// (5-D im2col loads), channel-major (NCHW) stores from the direct epilogue.
//
// Balanced schedule (KParams::sk): instead of whole tiles dealt out round-robin, the (tile, ring
// stage) pairs of the whole problem form one line of work units that is cut into equal runs, one
// per CTA pair.  A run starts and ends inside tiles, so a tile may be shared by two (seldom three)
// pairs, each holding a K range of it.  A pair takes its two shared tiles first (struct Walk).  The
// pair that holds the START of a tile's K range stores its partial sums into the output tile
// itself and raises a flag per epilogue warp; the pair that holds the range after it waits
// (bounded) for the flag, reads the partial sums back (they are still in L2), adds them to its
// accumulator and stores the result.  No atomics, no workspace, a fixed order of additions, and
// every pair does the same number of ring stages whatever the tile count.
//
// Every wait on an mbarrier is bounded.  When one runs out, the CTA raises a shared abort flag,
// every role leaves its loop, in-flight TMA loads and MMAs are waited for (bounded again), TMEM
// is freed and HB_ERR_TIMEOUT is left in the device status word.
#pragma once
#include "hb_ptx.cuh"
#include <cuda_fp16.h>
#include <type_traits>

namespace hb {

constexpr int kMaxStages = 12;
constexpr int kTileM = 128;
constexpr int kEpiWarps = 4;
constexpr int kThreads = 32 * (2 + kEpiWarps);       // strip conv kernel: producer, MMA, epilogue
constexpr int kEpiBufBytes = 4096;  // 32 rows x 128 bytes
// GEMM kernel: four epilogue warps (one per TMEM lane quadrant, two staging buffers each) or
// eight (two per quadrant, each with half of a tile's column chunks and one staging buffer),
// chosen per launch, and a second producer warp after them
constexpr int kUmmaEpiWarpsMax = 8;
constexpr int kUmmaEpiBytes = kUmmaEpiWarpsMax * kEpiBufBytes;
constexpr int kUmmaThreadsMax = 32 * (3 + kUmmaEpiWarpsMax);
__host__ __device__ constexpr int umma_threads(int epi_warps) { return 32 * (3 + epi_warps); }
constexpr int kErrTimeout = 5;      // HB_ERR_TIMEOUT

struct KParams {
  int M, N, K, batch;
  int BN, SW, esize_in, esize_out;
  int stages, acc_stages, tmem_cols;
  int kslices;  // 128-byte (swizzle-span) K slices behind one ring barrier: 1 or 2
  int tiles_m, tiles_n, num_tiles, num_kb;
  int raster, kind, b_mn_major, a_im2col, epilogue, l2_prefetch;
  int probe;            // diagnostic modes; only builds with -DHB_PROBES read it
  int epi_warps;        // epilogue warps of a CTA: 4 or 8
  // TMA-store epilogue: the same tile also goes to these outputs (other GPUs' copies of the output
  // buffer, reached over NVLink); tensor maps in this device's global memory
  const CUtensorMap* peer_maps;
  int n_peers;
  int silent_producer;  // test hook: the producers issue no loads, so the consumers' waits run out
  // Balanced schedule: work units are ring stages; unit u belongs to tile u / sk_per_tile.  CTA
  // pair i walks units [bound(i), bound(i+1)), bound(i) = i * sk_total / pairs, moved to the tile
  // edge when it falls closer to one than sk_min units.  flags then holds one int per (pair,
  // epilogue warp): "the partial sums of this pair's first, shared tile are in memory".
  int sk, sk_total, sk_per_tile, sk_min;
  // Tail balancing: the first `whole_tiles` tiles are 128*CG x BN; each remaining tile is cut into
  // `split` column slices of BN/split, so that the last, partly filled wave of the persistent
  // grid is made of shorter work items.  num_tiles counts work items (whole tiles + slices).
  int whole_tiles, split;
  // Alternatively (ksplit > 1, split == 1) each remaining tile is cut into `ksplit` slices of the
  // reduction: full-width work items whose epilogue adds into an output that was zeroed first.
  int ksplit;
  // kslab = 1 (with ksplit > 1 and whole_tiles == 0): slice s of every tile is stored, not added,
  // into slab s of a (ksplit, M, N) workspace; a later kernel sums the slabs in a fixed order.
  int kslab;
  // flags != nullptr (with ksplit > 1, no slabs): the K slices of a tile take turns instead of adding
  // into a zeroed output.  Slice 0 stores its partial sums, slice s > 0 waits until flags[tile] shows
  // that every epilogue warp of slice s-1 has finished, then adds its own.  No zeroing pass, and the
  // order of the additions is fixed.  The last arrival resets the flag for the next launch.
  int* flags;
  uint32_t idesc_split;
  long long wait_limit_cycles;  // 0: the default bound on every mbarrier wait
  uint32_t idesc;
  // conv geometry (a_im2col only)
  int HO, WO, KW, CI, kb_per_tap, stride_h, stride_w, dil_h, dil_w, pad_h, pad_w;
  // a_im2col == 2: 3-D convolution over an NDHWC tensor (5-D im2col loads); taps ordered (kd, kh, kw)
  int DO, KH, stride_d, pad_d;
  // direct-store epilogue
  int out_nchw;  // conv only: C is (N, CO, HO, WO) instead of (N*HO*WO, CO)
  int a_shared;  // batched: A has no batch dimension (every batch multiplies the same matrix)
  void* C;
  long long ldc;             // elements between consecutive rows of C
  long long batch_stride_c;  // elements between consecutive batches of C
};

// Device status word: HB_OK, or HB_ERR_TIMEOUT once any CTA gave up on a wait.
__device__ int g_hb_status = 0;

struct SmemBars {
  uint64_t full[kMaxStages];
  uint64_t empty[kMaxStages];
  uint64_t tmem_full[2];
  uint64_t tmem_empty[2];
  uint64_t drain;
  uint32_t tmem_base;
  int abort_flag;
};

// Bounded wait used while draining after an abort (ignores the abort flag).
__device__ __forceinline__ void mbar_wait_drain(uint32_t bar, uint32_t parity) {
  const long long t0 = clock64();
  while (!mbar_try_wait(bar, parity)) {
    if (clock64() - t0 > (HB_WAIT_LIMIT_CYCLES / 4)) return;
  }
}

// First work unit of CTA pair `i` of `n` under the balanced schedule: `total` units of
// `per_tile` ring stages per tile; a cut closer than `min_run` stages to a tile edge moves onto it.
__host__ __device__ __forceinline__ int sk_bound_of(int total, int per_tile, int min_run, int i, int n) {
  int b = static_cast<int>(static_cast<long long>(i) * total / n);
  const int r = b % per_tile;
  if (r != 0) {
    if (r < min_run) b -= r;
    else if (per_tile - r < min_run) b += per_tile - r;
  }
  return b;
}
__host__ __device__ __forceinline__ int sk_bound(const KParams& p, int i, int n) {
  return sk_bound_of(p.sk_total, p.sk_per_tile, p.sk_min, i, n);
}

// The work items of one CTA pair, in the order it takes them.  Static list: work items `unit`,
// `unit + n`, ...  Balanced schedule: the tiles its run [lo, hi) touches, the two shared ones
// FIRST — the run's last tile (of which it holds the first K stages: it stores partial sums for
// the next pair), then the run's first tile (of which it holds the last K stages: it adds what
// the pair before has stored) — and the whole tiles after them.  Both hand-overs thus happen at
// the start of a run, hidden behind the main loop of the tiles that follow, and the last thing
// every pair does is an ordinary tile.
struct Walk {
  int cur, end, step;  // static list: next item, item count, stride.  balanced: next whole tile, last + 1, phase
  int lo, hi;          // balanced: the run
};
struct Piece {
  int t;       // work item (static list) or tile (balanced schedule)
  int s0, s1;  // balanced schedule: ring stages [s0, s1) of the tile
};
__host__ __device__ __forceinline__ Walk walk_begin(const KParams& p, int unit, int n) {
  Walk w;
  if (p.sk) {
    w.lo = sk_bound(p, unit, n);
    w.hi = sk_bound(p, unit + 1, n);
    w.cur = (w.lo + p.sk_per_tile - 1) / p.sk_per_tile;  // first whole tile
    w.end = w.hi / p.sk_per_tile;                        // one past the last whole tile
    w.step = 0;                                          // phase: 0 = run's last tile, 1 = run's first tile, 2 = whole tiles
  } else {
    w.cur = unit;
    w.end = p.num_tiles;
    w.step = n;
    w.lo = w.hi = 0;
  }
  return w;
}
__host__ __device__ __forceinline__ bool walk_next(const KParams& p, Walk& w, Piece& pc) {
  if (!p.sk) {
    if (w.cur >= w.end) return false;
    pc.t = w.cur;
    pc.s0 = pc.s1 = 0;
    w.cur += w.step;
    return true;
  }
  const int per = p.sk_per_tile;
  if (w.step == 0) {
    w.step = 1;
    if (w.hi <= w.lo) {  // an empty run
      w.step = 2;
      w.cur = w.end;
      return false;
    }
    const int t_hi = w.hi / per, s_hi = w.hi - t_hi * per;
    if (s_hi > 0) {  // the run ends inside tile t_hi
      const int t_lo = w.lo / per;
      pc.t = t_hi;
      pc.s0 = (t_lo == t_hi) ? w.lo - t_lo * per : 0;  // (a run inside one tile is one piece)
      pc.s1 = s_hi;
      if (t_lo == t_hi) w.step = 2;
      return true;
    }
  }
  if (w.step == 1) {
    w.step = 2;
    const int t_lo = w.lo / per, s_lo = w.lo - t_lo * per;
    if (s_lo > 0) {  // the run starts inside tile t_lo
      pc.t = t_lo;
      pc.s0 = s_lo;
      pc.s1 = per;
      return true;
    }
  }
  if (w.cur >= w.end) return false;
  pc.t = w.cur++;
  pc.s0 = 0;
  pc.s1 = per;
  return true;
}

__device__ __forceinline__ uint4 ld_cg_v4(const void* ptr) {
  uint4 v;
  asm volatile("ld.global.cg.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(ptr)
               : "memory");
  return v;
}

// The tile in `buf` to every further output of the plan (tensor maps in global memory).
__device__ __noinline__ void tma_store_peers(const CUtensorMap* maps, int n, uint32_t buf, int col, int row, int z) {
  for (int r = 0; r < n; ++r) tma_store_3d(maps + r, buf, col, row, z);
}

// EW: epilogue warps of a CTA, 4 or 8.  A template parameter so that each form has its own launch
// bounds and drain loop: with the count a run-time value (or the drain in a generic lambda under
// the larger form's launch bounds) the four-warp form lost 10-30 % on short-K shapes.
template <int OUT_BYTES, int CG, int KIND, int KS, int EW = 4>
__global__ void __launch_bounds__(umma_threads(EW), 1)
hb_umma_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
               const __grid_constant__ CUtensorMap tmC, const __grid_constant__ CUtensorMap tmB2,
               const KParams p) {
  extern __shared__ uint8_t smem_raw[];
  // Swizzled TMA boxes and UMMA descriptors want 1024-byte aligned stage bases.
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (smem_base - smem_u32(smem_raw));

  const uint32_t cta_rank = (CG == 2) ? cluster_ctarank() : 0u;
  const bool leader = cta_rank == 0u;
  const int bn_cta = p.BN / CG;  // rows of B (columns of the tile) this CTA stages
  const int a_bytes = kTileM * p.SW;
  const int b_bytes = bn_cta * p.SW;
  const uint32_t sA = smem_base;
  constexpr int G = KS;  // K slices (swizzle spans) behind one ring barrier; equals p.kslices
  const uint32_t sB = sA + p.stages * G * a_bytes;
  // the epilogue staging buffers are 128-byte swizzled: 1024-byte aligned whatever the ring size
  const uint32_t sEpi = (sB + p.stages * G * b_bytes + 1023u) & ~1023u;
  const int epi_bytes = p.epilogue ? kUmmaEpiBytes : 0;
  SmemBars* bars = reinterpret_cast<SmemBars*>(smem + (sEpi - smem_base) + epi_bytes);
  volatile int* abort_flag = &bars->abort_flag;
  const WaitCtx wctx{abort_flag, p.wait_limit_cycles > 0 ? p.wait_limit_cycles : HB_WAIT_LIMIT_CYCLES};

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int BK = p.SW / p.esize_in;  // K elements per ring stage

  if (threadIdx.x == 0) {
    for (int s = 0; s < p.stages; ++s) {
      mbar_init(smem_u32(&bars->full[s]), 1);
      mbar_init(smem_u32(&bars->empty[s]), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(smem_u32(&bars->tmem_full[a]), 1);
      mbar_init(smem_u32(&bars->tmem_empty[a]), EW * CG);
    }
    mbar_init(smem_u32(&bars->drain), 1);
    bars->abort_flag = 0;
    fence_mbar_init();
    prefetch_tmap(&tmA);
    prefetch_tmap(&tmB);
    if (p.epilogue) prefetch_tmap(&tmC);
  }
  if (warp == 1) tmem_alloc_cg<CG>(smem_u32(&bars->tmem_base), static_cast<uint32_t>(p.tmem_cols));
  tc_fence_before();
  __syncthreads();
  if (CG == 2) cluster_sync();  // the peer's barriers exist before anything arrives on them
  tc_fence_after();
  const uint32_t tmem_base = bars->tmem_base;
  // Everything above touched only this CTA's own resources; the operands may still be being
  // written by the layout kernel this one was launched behind.
  griddep_wait();
  // A launch behind this one in the stream (made with programmatic serialization) may now take
  // SMs as this grid's CTAs leave them and set itself up; it waits, as above, for this grid to end.
  griddep_launch_dependents();

  const int tiles_per_batch = p.tiles_m * p.tiles_n;
  const int first_tile = blockIdx.x / CG;  // a pair of CTAs walks the tile list together
  const int tile_step = gridDim.x / CG;
  const int tile_rows = kTileM * CG;
  // work item -> (batch, first row of the pair tile, first column, width)
  auto decode = [&](const Piece& pc, int& b, int& m_pair, int& n_first, int& bn, int& kb0, int& kb1, int& kslice) {
    int t = pc.t;
    int slice = 0;
    bn = p.BN;
    kb0 = 0;
    kb1 = p.num_kb;
    kslice = 0;
    if (p.sk) {
      kb0 = pc.s0 * KS;
      kb1 = min(pc.s1 * KS, p.num_kb);
    } else if (t >= p.whole_tiles) {
      const int h = t - p.whole_tiles;
      if (p.ksplit > 1) {
        const int ks = h % p.ksplit;
        kslice = ks;
        t = p.whole_tiles + h / p.ksplit;
        kb0 = ks * p.num_kb / p.ksplit;
        kb1 = (ks + 1) * p.num_kb / p.ksplit;
      } else {
        slice = h % p.split;
        t = p.whole_tiles + h / p.split;
        bn = p.BN / p.split;
      }
    }
    b = t / tiles_per_batch;
    const int r = t - b * tiles_per_batch;
    const int mb = p.raster ? (r % p.tiles_m) : (r / p.tiles_n);
    const int nb = p.raster ? (r / p.tiles_m) : (r % p.tiles_n);
    m_pair = mb * tile_rows;
    n_first = nb * p.BN + slice * bn;
  };

  // part bit 0: the A operand (and the barrier's expect_tx); bit 1: the B operand
  auto produce = [&](int part) {
    int stage = 0;
    uint32_t phase = 0;
    long long issued = 0;
    bool ok = true;
    const int chunk_cols = p.SW / p.esize_in;               // MN-major B: columns per chunk
    // silent_producer (a test hook): nothing is loaded, so the consumers' bounded waits run out
    // and the abort path (drain, TMEM release, status word) is what the launch exercises
    Walk walk = walk_begin(p, first_tile, tile_step);
    Piece pc;
    while (ok && !p.silent_producer && walk_next(p, walk, pc)) {
      int b, m_pair, n_first, bn, kb0, kb1, kslice;
      decode(pc, b, m_pair, n_first, bn, kb0, kb1, kslice);
      const int bn_mine = bn / CG;  // B rows this CTA stages for this work item
      const int n_chunks = p.b_mn_major ? bn_mine / chunk_cols : 1;
      const uint32_t tx_bytes = static_cast<uint32_t>(a_bytes + bn_mine * p.SW) * CG;
      const CUtensorMap* tmBk = (bn == p.BN) ? &tmB : &tmB2;  // K-major B: box rows = bn / CG
      const int m0 = m_pair + static_cast<int>(cta_rank) * kTileM;
      const int n0 = n_first + static_cast<int>(cta_rank) * bn_mine;
      int pix_w = 0, pix_h = 0, pix_d = 0, pix_n = 0;
      if (p.a_im2col) {
        const int hw = p.HO * p.WO;
        int rem;
        if (p.a_im2col == 2) {
          const int dhw = p.DO * hw;
          pix_n = m0 / dhw;
          rem = m0 - pix_n * dhw;
          const int z = rem / hw;
          rem -= z * hw;
          pix_d = z * p.stride_d - p.pad_d;
        } else {
          pix_n = m0 / hw;
          rem = m0 - pix_n * hw;
        }
        const int y = rem / p.WO;
        const int x = rem - y * p.WO;
        pix_w = x * p.stride_w - p.pad_w;
        pix_h = y * p.stride_h - p.pad_h;
      }
      for (int kbg = kb0; kbg < kb1; kbg += G) {
        const int g = min(G, kb1 - kbg);  // K slices of this stage
        const uint32_t full_local = smem_u32(&bars->full[stage]);
        const uint32_t full = (CG == 2) ? mapa(full_local, 0) : full_local;  // the leader's barrier
        if (!mbar_wait(smem_u32(&bars->empty[stage]), phase ^ 1u, wctx)) {
          ok = false;
          break;
        }
#ifdef HB_PROBES
        if (p.probe == 1 && issued >= p.stages) {
          // diagnostic: operands stay as first loaded; only the barrier protocol runs
          if (leader && (part & 1)) mbar_arrive(full_local);  // one arrival per stage: the A producer's
          ++issued;
          if (++stage == p.stages) {
            stage = 0;
            phase ^= 1u;
          }
          continue;
        }
#endif
#ifdef HB_PROBES
        // diagnostic (wrong results): 3 = every other stage keeps the B operand of its previous use:
        // a quarter less operand traffic from L2 for the same MMA work
        const bool skip_b = p.probe == 3 && (issued & 1) && issued >= p.stages;
        if (leader && (part & 1))
          mbar_arrive_expect_tx(full_local, (skip_b ? static_cast<uint32_t>(a_bytes) * CG : tx_bytes) * static_cast<uint32_t>(g));
#else
        constexpr bool skip_b = false;
        if (leader && (part & 1)) mbar_arrive_expect_tx(full_local, tx_bytes * static_cast<uint32_t>(g));
#endif
        for (int j = 0; j < g; ++j) {
          const int kb = kbg + j;
          const uint32_t dA = sA + (stage * G + j) * a_bytes;
          const uint32_t dB = sB + (stage * G + j) * b_bytes;
          int krow;  // first K index of this block in B's K dimension
          if (p.a_im2col) {
            const int tap = kb / p.kb_per_tap;
            const int cc = kb - tap * p.kb_per_tap;
            int ryz = tap / p.KW;
            const int rx = tap - ryz * p.KW;
            if ((part & 1) && p.a_im2col == 2) {
              const int rz = ryz / p.KH;
              const int ry = ryz - rz * p.KH;
              tma_load_im2col_5d_cg<CG>(dA, &tmA, full, cc * BK, pix_w, pix_h, pix_d, pix_n,
                                        static_cast<uint16_t>(rx), static_cast<uint16_t>(ry),
                                        static_cast<uint16_t>(rz));
            } else if (part & 1) {
              tma_load_im2col_4d_cg<CG>(dA, &tmA, full, cc * BK, pix_w, pix_h, pix_n,
                                        static_cast<uint16_t>(rx * p.dil_w), static_cast<uint16_t>(ryz * p.dil_h));
            }
            krow = tap * p.CI + cc * BK;
          } else {
            if (part & 1) tma_load_3d_cg<CG>(dA, &tmA, full, kb * BK, m0, p.a_shared ? 0 : b);
            krow = kb * BK;
            if (p.l2_prefetch > 0 && kb + p.l2_prefetch < kb1) {
              tma_prefetch_3d(&tmA, (kb + p.l2_prefetch) * BK, m0, b);
              tma_prefetch_3d(tmBk, (kb + p.l2_prefetch) * BK, n0, b);
            }
          }
          if (!(part & 2) || skip_b) {
          } else if (p.b_mn_major) {
            for (int c = 0; c < n_chunks; ++c)
              tma_load_3d_cg<CG>(dB + c * (BK * p.SW), &tmB, full, n0 + c * chunk_cols, krow, b);
          } else {
            tma_load_3d_cg<CG>(dB, tmBk, full, krow, n0, b);
          }
        }
        ++issued;
        if (++stage == p.stages) {
          stage = 0;
          phase ^= 1u;
        }
      }
    }
    if (!ok) {
      // Wait (bounded) for the loads that are still in flight before shared memory goes away.
      // A full barrier completes only when both CTAs' loads of that stage have landed, so the
      // leader's wait covers the peer's copies too; the peer, which cannot poll the leader's
      // barrier, gives its own copies a fixed grace period instead.
      if (leader) {
        const int pending = issued < p.stages ? static_cast<int>(issued) : p.stages;
        for (int i = 0; i < pending; ++i) {
          if (--stage < 0) {
            stage = p.stages - 1;
            phase ^= 1u;
          }
          mbar_wait_drain(smem_u32(&bars->full[stage]), phase);
        }
      } else {
        const long long t0 = clock64();
        while (clock64() - t0 < 4000000LL) {
        }
      }
    }
      };
  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------------------
    // elect.sync (not "lane == 0") picks the issuing lane: the compiler then knows the branch
    // runs on exactly one lane and keeps descriptors and coordinates in uniform registers,
    // which is what the TMA and MMA instructions read their operands from.
    if (elect_one()) produce(1);
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------ MMA issuer (leader CTA only) ---------------------------
    if (elect_one() && leader) {
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      // Descriptors are built once per kernel (high word) and once per stage (low word); the
      // four MMAs of a stage differ only by a constant added to the 14-bit start-address field.
      const uint32_t layout_type = p.SW == 128 ? 2u : (p.SW == 64 ? 4u : 6u);
      const uint32_t sbo = 8u * p.SW;                // bytes between 8-row groups
      const int n_mma = p.SW / 32;                   // MMAs per ring stage (32 bytes of K each)
      const int umma_k = 32 / p.esize_in;            // 16 (fp16) or 32 (int8)
      const uint32_t b_lbo = p.b_mn_major ? static_cast<uint32_t>(BK * p.SW) : 16u;
      const uint32_t b_step16 = (p.b_mn_major ? static_cast<uint32_t>(umma_k * p.SW) : 32u) >> 4;
      const uint64_t desc_hi =
          static_cast<uint64_t>(((sbo >> 4) & 0x3FFFu) | (1u << 14) | (layout_type << 29)) << 32;
      const uint32_t a_lo_fixed = (16u >> 4) << 16;
      const uint32_t b_lo_fixed = ((b_lbo >> 4) & 0x3FFFu) << 16;
      const uint32_t idesc = p.idesc;
      const int num_kb = p.num_kb, stages = p.stages, acc_stages = p.acc_stages;
#ifdef HB_PROBES
      const int probe = p.probe;
#endif
      const uint32_t a16 = static_cast<uint32_t>(a_bytes) >> 4, b16 = static_cast<uint32_t>(b_bytes) >> 4;
      const uint32_t full0 = smem_u32(&bars->full[0]), empty0 = smem_u32(&bars->empty[0]);
      Walk walk = walk_begin(p, first_tile, tile_step);
      Piece pc;
      while (ok && walk_next(p, walk, pc)) {
        const int t = pc.t;
        if (!mbar_wait(smem_u32(&bars->tmem_empty[acc]), acc_phase ^ 1u, wctx)) {
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc * p.BN);
        const uint32_t idesc_t = (t >= p.whole_tiles) ? p.idesc_split : idesc;
        uint32_t accum = 0u;
        int n_kb = num_kb;  // K blocks of this work item
        if (p.sk) {
          n_kb = min(pc.s1 * G, num_kb) - pc.s0 * G;
        } else if (t >= p.whole_tiles && p.ksplit > 1) {
          const int ks = (t - p.whole_tiles) % p.ksplit;
          n_kb = (ks + 1) * num_kb / p.ksplit - ks * num_kb / p.ksplit;
        }
        for (int kbg = 0; kbg < n_kb; kbg += G) {
          const int g = min(G, n_kb - kbg);
          if (!mbar_wait(full0 + 8u * stage, phase, wctx)) {
            ok = false;
            break;
          }
          tc_fence_after();
          for (int j = 0; j < g; ++j) {
            const int slot = stage * G + j;
            uint32_t a_lo = (((sA >> 4) + slot * a16) & 0x3FFFu) | a_lo_fixed;
            uint64_t a_hi_extra = 0;
#ifdef HB_PROBES
            if (probe >= 16) {
              // diagnostic: start the A descriptor `shift` rows (128 bytes each) into the tile,
              // with (probe >= 32) or without the descriptor's base-offset field set
              const uint32_t shift = static_cast<uint32_t>(probe & 15);
              const uint32_t addr = sA + slot * a_bytes + shift * 128u;
              a_lo = ((addr >> 4) & 0x3FFFu) | a_lo_fixed;
              if (probe >= 32) a_hi_extra = static_cast<uint64_t>((addr >> 7) & 7u) << 49;
            }
            if (probe == 2) continue;  // diagnostic: loads only
#endif
            const uint32_t b_lo = (((sB >> 4) + slot * b16) & 0x3FFFu) | b_lo_fixed;
#pragma unroll
            for (int k = 0; k < 4; ++k) {
              if (k < n_mma) {
                umma_cg<CG, KIND>(d_tmem, desc_hi | a_hi_extra | (a_lo + 2u * k), desc_hi | (b_lo + b_step16 * k), idesc_t,
                                  accum);
                accum = 1u;
              }
            }
          }
          umma_commit_cg<CG>(empty0 + 8u * stage);  // stage reusable once these MMAs finish
          if (++stage == stages) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (!ok) break;
        umma_commit_cg<CG>(smem_u32(&bars->tmem_full[acc]));  // accumulator complete
        if (++acc == acc_stages) {
          acc = 0;
          acc_phase ^= 1u;
        }
      }
      if (!ok) {
        // Let every MMA issued so far finish before TMEM is freed.
        umma_commit_local<CG>(smem_u32(&bars->drain));
        mbar_wait_drain(smem_u32(&bars->drain), 0u);
      }
    }
    __syncwarp();
  } else if (warp >= 2 + EW) {
    // ------------------------------ second TMA producer: the B operand ---------------------
    if (elect_one()) produce(2);
    __syncwarp();
  } else {
    // ------------------------------ epilogue ----------------------------------------------
    constexpr bool kEight = EW == 8;
    constexpr int kWarps = EW;
    const int q = warp & 3;  // TMEM lane quadrant this warp may read
    const int ew = warp - 2;
    const int half = kEight ? (ew >> 2) : 0;  // with eight warps: which half of a tile's column chunks
    constexpr uint32_t n_bufs = kUmmaEpiWarpsMax / kWarps;  // staging buffers of a warp
    uint32_t store_it = 0;
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    constexpr int kColsPerStore = 128 / OUT_BYTES;  // 32 (4-byte) or 64 (fp16) columns
    const uint32_t my_buf = sEpi + ew * n_bufs * kEpiBufBytes;
    Walk walk = walk_begin(p, first_tile, tile_step);
    Piece pc;
    while (ok && walk_next(p, walk, pc)) {
      const int t = pc.t;
      int b, m_pair, n0, bn, kb0, kb1, kslice;
      decode(pc, b, m_pair, n0, bn, kb0, kb1, kslice);
      // balanced schedule: does another pair hold the K stages after this piece's (it then stores
      // partial sums for that pair), or the ones before (it then adds that pair's partial sums)?
#ifdef HB_PROBES
      // diagnostics (wrong results): 21 = pieces written independently, no hand-over at all;
      // 22 = flags but no partial-sum loads; 23 = no wait for the partial stores before the flag
      const bool sk_prod = OUT_BYTES == 4 && p.sk && pc.s1 < p.sk_per_tile && p.probe != 21;
      const bool sk_cons = OUT_BYTES == 4 && p.sk && pc.s0 > 0 && p.probe != 21;
#else
      const bool sk_prod = OUT_BYTES == 4 && p.sk && pc.s1 < p.sk_per_tile;
      const bool sk_cons = OUT_BYTES == 4 && p.sk && pc.s0 > 0;
#endif
      const int sk_slot = static_cast<int>(cta_rank) * kWarps + ew;
      const bool ksliced = OUT_BYTES == 4 && p.ksplit > 1 && t >= p.whole_tiles && !p.kslab;
      const bool chain = ksliced && p.flags != nullptr;
      const bool reduce = ksliced && (!chain || kslice > 0);
      int* const flag = chain ? p.flags + (t - p.whole_tiles) / p.ksplit : nullptr;
      constexpr int kArrivals = kWarps * CG;  // epilogue warps that work on one tile
      const int zc = p.kslab ? kslice : b;  // third coordinate of the output: batch, or workspace slab
      const int row0 = m_pair + static_cast<int>(cta_rank) * kTileM + q * 32;
      if (!mbar_wait_relaxed(smem_u32(&bars->tmem_full[acc]), acc_phase, wctx)) {
        ok = false;
        break;
      }
      tc_fence_after();
      if (sk_cons) {
        // The pair before this one took the tile first and left the sums of the earlier K stages in
        // the output: wait (bounded) until its warp for these 32 rows says they are in memory.
        const int* f = p.flags + first_tile * kArrivals + sk_slot;
        int got = 1;
        if (lane == 0) {
          const long long t0 = clock64();
          while (ld_acquire_gpu(f) == 0) {
            if (*abort_flag || clock64() - t0 > wctx.limit_cycles) {
              *abort_flag = 1;
              got = 0;
              break;
            }
            __nanosleep(64);
          }
        }
        got = __shfl_sync(0xffffffffu, got, 0);
        __syncwarp();
        if (!got) {
          ok = false;
          break;
        }
      }
      if (chain && kslice > 0) {
        // wait (bounded) for the slice before this one to have written the tile
        int got = 1;
        if (lane == 0) {
          const long long t0 = clock64();
          while (ld_acquire_gpu(flag) < kslice * kArrivals) {
            if (*abort_flag || clock64() - t0 > wctx.limit_cycles) {
              *abort_flag = 1;
              got = 0;
              break;
            }
            __nanosleep(64);
          }
        }
        got = __shfl_sync(0xffffffffu, got, 0);
        if (!got) {
          ok = false;
          break;
        }
        fence_proxy_async_all();
      }
      const uint32_t t_addr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) +
                              static_cast<uint32_t>(acc * p.BN);
      // Software pipeline over 128-byte column chunks: the TMEM load of chunk i+1 is in flight
      // while chunk i goes through shared memory to its TMA store.
      // Two warps of a quadrant split the chunks: the first takes the lower half (the larger
      // one when the count is odd), the second the rest, which may be nothing.
      const int n_chunks = (bn + kColsPerStore - 1) / kColsPerStore;
      const int c_mid = !kEight ? bn : min(bn, ((n_chunks + 1) >> 1) * kColsPerStore);
      const int c_lo = half ? c_mid : 0;
      const int c_hi = half ? bn : c_mid;
      uint32_t v[32];
      uint32_t v2[OUT_BYTES == 2 ? 32 : 1];
      if (!kEight || c_lo < c_hi) {
        tmem_ld_32x32(t_addr + c_lo, v);
        if (OUT_BYTES == 2) tmem_ld_32x32(t_addr + c_lo + 32, reinterpret_cast<uint32_t(&)[32]>(v2));
      } else {
        // no chunk for this warp: the accumulator is handed back at once
        tc_fence_before();
        __syncwarp();
        if (lane == 0) {
          if (CG == 2)
            mbar_arrive_cluster(mapa(smem_u32(&bars->tmem_empty[acc]), 0));
          else
            mbar_arrive(smem_u32(&bars->tmem_empty[acc]));
        }
      }
      // balanced schedule, consumer piece: this thread's 128 bytes of the partial sums another
      // pair left in the output, for the column chunk that starts at tile column c (zeros where
      // the tile hangs over the edge of C; rows are 16-byte multiples: whole vectors or none)
      uint4 part[OUT_BYTES == 4 ? 8 : 1];
      auto load_part = [&](int c) {
        const int row = row0 + lane, col = n0 + c;
        const uint8_t* src = static_cast<const uint8_t*>(p.C) +
                             (static_cast<long long>(b) * p.batch_stride_c +
                              static_cast<long long>(row) * p.ldc + col) * 4;
#pragma unroll
        for (int j = 0; j < (OUT_BYTES == 4 ? 8 : 1); ++j) {
#ifdef HB_PROBES
          if (p.probe == 22) {
            part[j] = make_uint4(0u, 0u, 0u, 0u);
            continue;
          }
#endif
          if (row < p.M && col + 4 * j < p.N)
            part[j] = ld_cg_v4(src + 16 * j);
          else
            part[j] = make_uint4(0u, 0u, 0u, 0u);
        }
      };
      if (OUT_BYTES == 4 && sk_cons && c_lo < c_hi) load_part(c_lo);
      for (int c0 = c_lo; c0 < c_hi; c0 += kColsPerStore) {
        uint32_t packed[32];  // 128 bytes of output for this thread's row
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
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            __half2 h = __floats2half2_rn(__uint_as_float(v2[(2 * i) % (OUT_BYTES == 2 ? 32 : 1)]),
                                          __uint_as_float(v2[(2 * i + 1) % (OUT_BYTES == 2 ? 32 : 1)]));
            packed[16 + i] = *reinterpret_cast<uint32_t*>(&h);
          }
        }
        if constexpr (OUT_BYTES == 4) {
          if (sk_cons) {
            // add the other pair's partial sums (fetched one chunk ahead), then start the next fetch
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              if (KIND == 1) {
                packed[4 * j] += part[j].x; packed[4 * j + 1] += part[j].y;
                packed[4 * j + 2] += part[j].z; packed[4 * j + 3] += part[j].w;
              } else {
                packed[4 * j] = __float_as_uint(__uint_as_float(packed[4 * j]) + __uint_as_float(part[j].x));
                packed[4 * j + 1] = __float_as_uint(__uint_as_float(packed[4 * j + 1]) + __uint_as_float(part[j].y));
                packed[4 * j + 2] = __float_as_uint(__uint_as_float(packed[4 * j + 2]) + __uint_as_float(part[j].z));
                packed[4 * j + 3] = __float_as_uint(__uint_as_float(packed[4 * j + 3]) + __uint_as_float(part[j].w));
              }
            }
            if (c0 + kColsPerStore < c_hi) load_part(c0 + kColsPerStore);
          }
        }
        if (c0 + kColsPerStore < c_hi) {
          tmem_ld_32x32(t_addr + c0 + kColsPerStore, v);
          if (OUT_BYTES == 2)
            tmem_ld_32x32(t_addr + c0 + kColsPerStore + 32, reinterpret_cast<uint32_t(&)[32]>(v2));
        }
        if (c0 + kColsPerStore >= c_hi) {
          // Last read of this accumulator: hand it back to the MMA warp before storing.
          tc_fence_before();
          __syncwarp();
          if (lane == 0) {
            if (CG == 2)
              mbar_arrive_cluster(mapa(smem_u32(&bars->tmem_empty[acc]), 0));
            else
              mbar_arrive(smem_u32(&bars->tmem_empty[acc]));
          }
        }
        const int col = n0 + c0;
        if (p.epilogue) {
          if (col < p.N && row0 < p.M) {
            const uint32_t buf = my_buf + (n_bufs == 2 ? (store_it & 1u) * kEpiBufBytes : 0u);
            ++store_it;
            const bool issuer = elect_one();
            // the store that last used this buffer has read it (every lane waits: only the one
            // that issued stores has groups to wait for)
            if (n_bufs == 2)
              bulk_wait_read<1>();
            else
              bulk_wait_read<0>();
            __syncwarp();
            const uint32_t row_addr = buf + lane * 128;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              const uint32_t a = row_addr + ((j ^ (lane & 7)) << 4);
              asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(a), "r"(packed[4 * j]),
                           "r"(packed[4 * j + 1]), "r"(packed[4 * j + 2]), "r"(packed[4 * j + 3])
                           : "memory");
            }
            fence_proxy_async_smem();
            __syncwarp();
            if (issuer) {
              if (reduce)
                tma_reduce_add_3d(&tmC, buf, col, row0, zc);
              else
                tma_store_3d(&tmC, buf, col, row0, zc);
              bulk_commit();
              // (plain stores into other GPUs' memory, a bulk group of their own: nothing here waits
              // on a peer; the waits on this buffer's earlier groups count groups in order, so one
              // more group per chunk only makes them wait for more)
              if (p.n_peers) {
                tma_store_peers(p.peer_maps, p.n_peers, buf, col, row0, zc);
                bulk_commit();
              }
            }
          }
        } else {
          const int row = row0 + lane;
          if (row < p.M && col < p.N) {
            uint8_t* base = static_cast<uint8_t*>(p.C) +
                            (static_cast<long long>(zc) * p.batch_stride_c +
                             static_cast<long long>(row) * p.ldc + col) *
                                OUT_BYTES;
            const bool vec_ok = ((reinterpret_cast<uintptr_t>(base) & 15u) == 0) &&
                                (col + kColsPerStore <= p.N);
            if (p.out_nchw) {
              // channel-major output: for one channel the 32 lanes of the warp hold 32 consecutive
              // pixels, so each store instruction writes one contiguous run (two where the warp
              // straddles two images)
              const int P = p.HO * p.WO * (p.a_im2col == 2 ? p.DO : 1);
              const int n = row / P;
              const int pix = row - n * P;
              uint8_t* o = static_cast<uint8_t*>(p.C) +
                           ((static_cast<long long>(n) * p.N + col) * P + pix) * OUT_BYTES;
              const long long cstep = static_cast<long long>(P) * OUT_BYTES;
              const int ncols = min(kColsPerStore, p.N - col);
#pragma unroll
              for (int i = 0; i < kColsPerStore; ++i) {
                if (i < ncols) {
                  if (OUT_BYTES == 4)
                    *reinterpret_cast<uint32_t*>(o + i * cstep) = packed[i % 32];
                  else
                    *reinterpret_cast<uint16_t*>(o + i * cstep) =
                        static_cast<uint16_t>(packed[(i >> 1) % 32] >> (16 * (i & 1)));
                }
              }
            } else if (reduce) {
              const int ncols = min(kColsPerStore, p.N - col);
#pragma unroll
              for (int i = 0; i < 32; ++i) {
                if (i < ncols) {
                  if (KIND == 1)
                    atomicAdd(reinterpret_cast<int*>(base) + i, static_cast<int>(packed[i]));
                  else
                    atomicAdd(reinterpret_cast<float*>(base) + i, __uint_as_float(packed[i]));
                }
              }
            } else if (vec_ok) {
#pragma unroll
              for (int j = 0; j < 8; ++j) {
                *reinterpret_cast<uint4*>(base + 16 * j) =
                    make_uint4(packed[4 * j], packed[4 * j + 1], packed[4 * j + 2], packed[4 * j + 3]);
              }
            } else {
              const int ncols = min(kColsPerStore, p.N - col);
              if (OUT_BYTES == 4) {
                uint32_t* o = reinterpret_cast<uint32_t*>(base);
#pragma unroll
                for (int i = 0; i < 32; ++i)
                  if (i < ncols) o[i] = packed[i];
              } else {
                uint16_t* o = reinterpret_cast<uint16_t*>(base);
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                  if (2 * i < ncols) o[2 * i] = static_cast<uint16_t>(packed[i] & 0xFFFFu);
                  if (2 * i + 1 < ncols) o[2 * i + 1] = static_cast<uint16_t>(packed[i] >> 16);
                }
              }
            }
          }
        }
      }
      if (sk_prod || sk_cons) {
        // (the partial sums read above are in registers or already stored: the flag that
        // announced them goes back to zero for the next launch; then, if a later K range of this
        // tile is another pair's, this warp's rows are announced to it in turn)
#ifdef HB_PROBES
        if (sk_prod && p.epilogue && p.probe != 23) {
#else
        if (sk_prod && p.epilogue) {
#endif
          bulk_wait<0>();
          fence_proxy_async_all();
        }
        __syncwarp();
        if (lane == 0) {
          if (sk_cons) *(volatile int*)(p.flags + first_tile * kArrivals + sk_slot) = 0;
          if (sk_prod) {
            __threadfence();
            st_release_gpu(p.flags + (first_tile + 1) * kArrivals + sk_slot, 1);
          }
        }
      }
      if (chain) {
        // this warp's part of the tile is in memory: tell the next slice, or, as the very last
        // arrival of the tile, put the flag back to zero
        if (p.epilogue) bulk_wait<0>();
        __syncwarp();
        if (lane == 0) {
          __threadfence();
          if (atomicAdd(flag, 1) + 1 == p.ksplit * kArrivals) atomicExch(flag, 0);
        }
      }
      if (++acc == p.acc_stages) {
        acc = 0;
        acc_phase ^= 1u;
      }
    }
    // the lane that issued this warp's stores drains their groups (a no-op for the others):
    // shared memory must outlive the stores' reads of it; their writes complete with the grid
    if (p.epilogue) bulk_wait_read<0>();
    __syncwarp();
  }

  tc_fence_before();
  __syncthreads();
  if (CG == 2) cluster_sync();  // neither CTA leaves while the other may still touch its barriers
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_cg<CG>(tmem_base, static_cast<uint32_t>(p.tmem_cols));
  }
  if (threadIdx.x == 0 && *abort_flag) atomicExch(&g_hb_status, kErrTimeout);
}

}  // namespace hb
