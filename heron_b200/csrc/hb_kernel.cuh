// The one kernel body behind GEMM, batched GEMM and NHWC conv2d (implicit GEMM).
//
//   D[b, m, n] = sum_k A[b, m, k] * B[b, n, k]
//
// Persistent CTAs (one per SM) walk a static list of 128 x BN output tiles.  Inside a CTA the
// warps have fixed roles:
//   warp 0      one elected lane issues TMA loads into a ring of shared-memory stages;
//   warp 1      allocates TMEM; one elected lane issues tcgen05.mma into a TMEM accumulator and
//               commits stage-free / accumulator-full events to mbarriers;
//   warps 2..5  epilogue: tcgen05.ld the accumulator (each warp owns the 32 TMEM lanes its
//               position in the warpgroup may touch), convert, and write the tile either through
//               swizzled shared memory + TMA store or with direct vector stores.
// Two accumulator buffers in TMEM let the MMA warp start the next tile while the epilogue warps
// drain the previous one.
//
// Operand layouts in shared memory are the canonical swizzled UMMA layouts, written by TMA:
//   A, K-major:   rows = M index, each row SW bytes of K (SW = 32/64/128 = TMA swizzle span);
//   B, K-major:   rows = N index, same (GEMM / BMM: B is stored (N, K));
//   B, MN-major:  rows = K index, each row SW bytes of N; BN*esize/SW such column chunks
//                 (conv: the HWIO filter is a (KH*KW*CI, CO) matrix with CO contiguous).
// For conv the A tile is fetched with im2col-mode TMA: 128 consecutive output pixels of one
// filter tap and one channel chunk, zero-filled where the tap falls into the padding.
//
// Every wait on an mbarrier is bounded.  When one runs out, the CTA raises a shared abort flag,
// every role leaves its loop, in-flight TMA loads and MMAs are waited for (bounded again), TMEM
// is freed and HB_ERR_TIMEOUT is left in the device status word.
#pragma once
#include "hb_ptx.cuh"
#include <cuda_fp16.h>

namespace hb {

constexpr int kMaxStages = 12;
constexpr int kTileM = 128;
constexpr int kEpiWarps = 4;
constexpr int kThreads = 32 * (2 + kEpiWarps);
constexpr int kEpiBufBytes = 4096;  // 32 rows x 128 bytes
constexpr int kErrTimeout = 5;      // HB_ERR_TIMEOUT

struct KParams {
  int M, N, K, batch;
  int BN, SW, esize_in, esize_out;
  int stages, acc_stages, tmem_cols;
  int tiles_m, tiles_n, num_tiles, num_kb;
  int raster, kind, b_mn_major, a_im2col, epilogue;
  uint32_t idesc;
  // conv geometry (a_im2col only)
  int HO, WO, KW, CI, kb_per_tap, stride_h, stride_w, dil_h, dil_w, pad;
  // direct-store epilogue
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

template <int OUT_BYTES>
__global__ void __launch_bounds__(kThreads, 1)
hb_umma_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
               const __grid_constant__ CUtensorMap tmC, const KParams p) {
  extern __shared__ uint8_t smem_raw[];
  // Swizzled TMA boxes and UMMA descriptors want 1024-byte aligned stage bases.
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (smem_base - smem_u32(smem_raw));

  const int a_bytes = kTileM * p.SW;
  const int b_bytes = p.BN * p.SW;
  const uint32_t sA = smem_base;
  const uint32_t sB = sA + p.stages * a_bytes;
  const uint32_t sEpi = sB + p.stages * b_bytes;
  const int epi_bytes = p.epilogue ? kEpiWarps * 2 * kEpiBufBytes : 0;
  SmemBars* bars = reinterpret_cast<SmemBars*>(smem + (sEpi - smem_base) + epi_bytes);
  volatile int* abort_flag = &bars->abort_flag;

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
      mbar_init(smem_u32(&bars->tmem_empty[a]), kEpiWarps);
    }
    mbar_init(smem_u32(&bars->drain), 1);
    bars->abort_flag = 0;
    fence_mbar_init();
    prefetch_tmap(&tmA);
    prefetch_tmap(&tmB);
    if (p.epilogue) prefetch_tmap(&tmC);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(&bars->tmem_base), static_cast<uint32_t>(p.tmem_cols));
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = bars->tmem_base;

  const int tiles_per_batch = p.tiles_m * p.tiles_n;

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      long long issued = 0;
      bool ok = true;
      const int chunk_cols = p.SW / p.esize_in;               // MN-major B: columns per chunk
      const int n_chunks = p.b_mn_major ? p.BN / chunk_cols : 1;
      const uint32_t tx_bytes = static_cast<uint32_t>(a_bytes + b_bytes);
      for (int t = blockIdx.x; ok && t < p.num_tiles; t += gridDim.x) {
        const int b = t / tiles_per_batch;
        const int r = t - b * tiles_per_batch;
        const int mb = p.raster ? (r % p.tiles_m) : (r / p.tiles_n);
        const int nb = p.raster ? (r / p.tiles_m) : (r % p.tiles_n);
        const int m0 = mb * kTileM;
        const int n0 = nb * p.BN;
        int pix_w = 0, pix_h = 0, pix_n = 0;
        if (p.a_im2col) {
          const int hw = p.HO * p.WO;
          pix_n = m0 / hw;
          const int rem = m0 - pix_n * hw;
          const int y = rem / p.WO;
          const int x = rem - y * p.WO;
          pix_w = x * p.stride_w - p.pad;
          pix_h = y * p.stride_h - p.pad;
        }
        for (int kb = 0; kb < p.num_kb; ++kb) {
          const uint32_t full = smem_u32(&bars->full[stage]);
          if (!mbar_wait(smem_u32(&bars->empty[stage]), phase ^ 1u, abort_flag)) {
            ok = false;
            break;
          }
          mbar_arrive_expect_tx(full, tx_bytes);
          const uint32_t dA = sA + stage * a_bytes;
          const uint32_t dB = sB + stage * b_bytes;
          int krow;  // first K index of this block in B's K dimension
          if (p.a_im2col) {
            const int tap = kb / p.kb_per_tap;
            const int cc = kb - tap * p.kb_per_tap;
            const int ry = tap / p.KW;
            const int rx = tap - ry * p.KW;
            tma_load_im2col_4d(dA, &tmA, full, cc * BK, pix_w, pix_h, pix_n,
                               static_cast<uint16_t>(rx * p.dil_w),
                               static_cast<uint16_t>(ry * p.dil_h));
            krow = tap * p.CI + cc * BK;
          } else {
            tma_load_3d(dA, &tmA, full, kb * BK, m0, b);
            krow = kb * BK;
          }
          if (p.b_mn_major) {
            for (int j = 0; j < n_chunks; ++j)
              tma_load_3d(dB + j * (BK * p.SW), &tmB, full, n0 + j * chunk_cols, krow, b);
          } else {
            tma_load_3d(dB, &tmB, full, krow, n0, b);
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
        const int pending = issued < p.stages ? static_cast<int>(issued) : p.stages;
        for (int i = 0; i < pending; ++i) {
          if (--stage < 0) {
            stage = p.stages - 1;
            phase ^= 1u;
          }
          mbar_wait_drain(smem_u32(&bars->full[stage]), phase);
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------ MMA issuer --------------------------------------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      const uint32_t layout_type = p.SW == 128 ? 2u : (p.SW == 64 ? 4u : 6u);
      const uint32_t sbo = 8u * p.SW;                // bytes between 8-row groups
      const int n_mma = p.SW / 32;                   // MMAs per ring stage (32 bytes of K each)
      const int umma_k = 32 / p.esize_in;            // 16 (fp16) or 32 (int8)
      const uint32_t b_lbo = p.b_mn_major ? static_cast<uint32_t>(BK * p.SW) : 16u;
      const uint32_t b_step = p.b_mn_major ? static_cast<uint32_t>(umma_k * p.SW) : 32u;
      for (int t = blockIdx.x; ok && t < p.num_tiles; t += gridDim.x) {
        if (!mbar_wait(smem_u32(&bars->tmem_empty[acc]), acc_phase ^ 1u, abort_flag)) {
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc * p.BN);
        for (int kb = 0; kb < p.num_kb; ++kb) {
          if (!mbar_wait(smem_u32(&bars->full[stage]), phase, abort_flag)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t aA = sA + stage * a_bytes;
          const uint32_t aB = sB + stage * b_bytes;
          for (int k = 0; k < n_mma; ++k) {
            const uint64_t adesc = make_smem_desc(aA + k * 32u, 16u, sbo, layout_type);
            const uint64_t bdesc = make_smem_desc(aB + k * b_step, b_lbo, sbo, layout_type);
            const uint32_t accum = (kb | k) != 0 ? 1u : 0u;
            if (p.kind == 0)
              umma_f16(d_tmem, adesc, bdesc, p.idesc, accum);
            else
              umma_i8(d_tmem, adesc, bdesc, p.idesc, accum);
          }
          umma_commit(smem_u32(&bars->empty[stage]));  // stage reusable once these MMAs finish
          if (++stage == p.stages) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (!ok) break;
        umma_commit(smem_u32(&bars->tmem_full[acc]));  // accumulator complete
        if (++acc == p.acc_stages) {
          acc = 0;
          acc_phase ^= 1u;
        }
      }
      if (!ok) {
        // Let every MMA issued so far finish before TMEM is freed.
        umma_commit(smem_u32(&bars->drain));
        mbar_wait_drain(smem_u32(&bars->drain), 0u);
      }
    }
    __syncwarp();
  } else {
    // ------------------------------ epilogue ----------------------------------------------
    const int q = warp & 3;  // TMEM lane quadrant this warp may read
    const int ew = warp - 2;
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    uint32_t store_it = 0;
    constexpr int kColsPerStore = 128 / OUT_BYTES;  // 32 (4-byte) or 64 (fp16) columns
    const uint32_t my_buf = sEpi + ew * 2 * kEpiBufBytes;
    for (int t = blockIdx.x; ok && t < p.num_tiles; t += gridDim.x) {
      const int b = t / tiles_per_batch;
      const int r = t - b * tiles_per_batch;
      const int mb = p.raster ? (r % p.tiles_m) : (r / p.tiles_n);
      const int nb = p.raster ? (r / p.tiles_m) : (r % p.tiles_n);
      const int row0 = mb * kTileM + q * 32;
      const int n0 = nb * p.BN;
      if (!mbar_wait(smem_u32(&bars->tmem_full[acc]), acc_phase, abort_flag)) {
        ok = false;
        break;
      }
      tc_fence_after();
      const uint32_t t_addr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) +
                              static_cast<uint32_t>(acc * p.BN);
      for (int c0 = 0; c0 < p.BN; c0 += kColsPerStore) {
        uint32_t v[32];
        uint32_t packed[32];  // 128 bytes of output for this thread's row
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
        if (c0 + kColsPerStore >= p.BN) {
          // Last read of this accumulator: hand it back to the MMA warp before storing.
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(smem_u32(&bars->tmem_empty[acc]));
        }
        const int col = n0 + c0;
        if (p.epilogue) {
          if (col < p.N && row0 < p.M) {
            const uint32_t buf = my_buf + (store_it & 1u) * kEpiBufBytes;
            ++store_it;
            if (lane == 0) bulk_wait_read<1>();  // the store that last used this buffer has read it
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
            if (lane == 0) {
              tma_store_3d(&tmC, buf, col, row0, b);
              bulk_commit();
            }
          }
        } else {
          const int row = row0 + lane;
          if (row < p.M && col < p.N) {
            uint8_t* base = static_cast<uint8_t*>(p.C) +
                            (static_cast<long long>(b) * p.batch_stride_c +
                             static_cast<long long>(row) * p.ldc + col) *
                                OUT_BYTES;
            const bool vec_ok = ((reinterpret_cast<uintptr_t>(base) & 15u) == 0) &&
                                (col + kColsPerStore <= p.N);
            if (vec_ok) {
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
      if (++acc == p.acc_stages) {
        acc = 0;
        acc_phase ^= 1u;
      }
    }
    if (p.epilogue && lane == 0) bulk_wait<0>();
    __syncwarp();
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, static_cast<uint32_t>(p.tmem_cols));
  }
  if (threadIdx.x == 0 && *abort_flag) atomicExch(&g_hb_status, kErrTimeout);
}

// Unpacks the x86 operator's int8 filter (CO/sco, KH, KW, CI/4, sco, 4) to HWIO (KH,KW,CI,CO).
// One thread per 4-byte group of input channels; consecutive threads walk output channels so
// that the HWIO writes of a warp land in consecutive bytes of four rows.
__global__ void hb_unpack_filter_kernel(const int8_t* __restrict__ packed, int8_t* __restrict__ hwio,
                                        int CO, int KH, int KW, int CI, int sco) {
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

}  // namespace hb
