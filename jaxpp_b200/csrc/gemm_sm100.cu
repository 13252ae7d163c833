// bf16 GEMM for sm_100a: D[M,N] = A[M,K] * B[N,K]^T with fp32 accumulation in tensor memory.
//
// One persistent CTA per SM walks 128x256 output tiles.  Warp 0 streams operand tiles into a 4-stage
// shared-memory ring with TMA (128-byte swizzle), warp 1 issues tcgen05.mma (128x256x16 per instruction)
// into one of two 256-column TMEM accumulators, warps 2-5 drain the other accumulator with tcgen05.ld
// and write the result (optionally + bias, optionally accumulated onto an existing fp32 D), so the
// epilogue of tile i overlaps the main loop of tile i+1.
//
// Either operand can be K-major (reduction dimension contiguous in memory) or MN-major (row/column
// dimension contiguous), which covers the three GEMMs of a linear layer without a transpose pass:
//   forward  y  = x  * w^T : A = x  (K-major),  B = w (K-major)
//   dgrad    dx = dy * w   : A = dy (K-major),  B = w (MN-major)
//   wgrad    dw = dy^T * x : A = dy (MN-major), B = x (MN-major)
// Every wait is bounded; on a time-out the kernel records a status, drains its own TMA copies, frees its
// tensor memory and returns.
#include "common.cuh"

#include <mutex>
#include <unordered_map>

namespace jpb {

constexpr int BM = 128, BN = 256, BK = 64, UMMA_K = 16;
constexpr int STAGES = 4;
constexpr int A_BYTES = BM * BK * 2;  // 16 KiB
constexpr int B_BYTES = BN * BK * 2;  // 32 KiB
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int GEMM_THREADS = 192;
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*alignment slack*/ + 256 /*barriers*/;
constexpr int TMEM_COLS = 512;

struct GemmParams {
  int M, N, K;
  int ldd;             // elements between rows of D
  int out_fp32;        // D is fp32 (else bf16)
  int accumulate;      // D += result (D must be fp32)
  int bias_fp32;
  const void* bias;    // per-column bias or nullptr
  void* D;
  int* status;
  int tiles_m, tiles_n;
  int a_blocked, b_blocked;  // MN-major operand addressed through a 3-D map {64, K, MN/64}: one copy per stage
  // Batched (grouped, equal-sized groups): `batch` problems stacked along the rows of each operand's storage --
  // A [batch*M, K] or [batch*K, M], B [batch*N, K] or [batch*K, N], D [batch*M, N].  Tiles that straddle the
  // end of a problem read rows of the next one; the epilogue masks them (and K must be a multiple of 64).
  int batch;
  int a_off, b_off;          // storage rows per problem of A and B
  // Groups of unequal size inside equal-sized storage: the M rows of a problem (count_k == 0) or its K reduction
  // rows (count_k == 1) are `segs` segments of `seg_rows` rows, and only the first counts[prob * segs + s] rows of
  // segment s hold data (the others are zero).  Output tiles, or 64-row reduction blocks, without a live row are
  // not loaded and not multiplied; an output tile without any is written as zeros (left alone when accumulating).
  const int* counts;         // device memory, or nullptr: every row is live
  int seg_rows, segs, count_k;
};

// Does [lo, hi) of problem `prob` contain a live row?  Every role of the CTA asks the same question about the same
// ranges and gets the same answer (the counts do not change while the kernel runs), so they skip in step.
__device__ __forceinline__ bool range_live(const GemmParams& p, int prob, int lo, int hi) {
  const int* c = p.counts + prob * p.segs;
  int q1 = (hi - 1) / p.seg_rows;
  if (q1 >= p.segs) q1 = p.segs - 1;
  for (int q = lo / p.seg_rows; q <= q1; ++q) {
    const int s = q * p.seg_rows;
    const int e = s + min(__ldg(c + q), p.seg_rows);
    if (e > s && lo < e && hi > s) return true;
  }
  return false;
}
// Is output tile [m0, m0 + BM) of problem `prob` worth computing?
__device__ __forceinline__ bool tile_live(const GemmParams& p, int prob, int m0) {
  if (p.counts == nullptr) return true;
  return p.count_k ? range_live(p, prob, 0, p.K) : range_live(p, prob, m0, m0 + BM);
}
// The 64-row reduction blocks of a problem that hold data, as a sequence of ranges [lo, hi): one range covering all
// k blocks when the counts do not describe K; otherwise one per non-empty segment (a block shared by two segments is
// visited once).  Every role walks the same sequence.  No division: this runs once per k block in the threads that
// issue the copies and the MMAs.
struct KRanges {
  int q = 0, next = 0, seg_lo = 0;
  __device__ __forceinline__ bool get(const GemmParams& p, int prob, int k_blocks, int& lo, int& hi) {
    if (p.counts == nullptr || !p.count_k) {
      if (q++ > 0) return false;
      lo = 0; hi = k_blocks;
      return true;
    }
    const int* c = p.counts + prob * p.segs;
    for (; q < p.segs; ++q, seg_lo += p.seg_rows) {
      const int n = min(__ldg(c + q), p.seg_rows);
      if (n <= 0) continue;
      lo = max(next, seg_lo / BK);
      hi = min(k_blocks, (seg_lo + n + BK - 1) / BK);
      if (lo >= hi) continue;
      next = hi;
      ++q; seg_lo += p.seg_rows;
      return true;
    }
    return false;
  }
};

// Tile rasterisation: groups of GROUP_M row blocks are walked column by column, so that the ~148 tiles in
// flight at any time touch about GROUP_M row panels of A and 148/GROUP_M column panels of B -- a working set that
// stays in L2 instead of re-streaming all of A for every column of tiles.
// With live-row counts the group is 15 blocks high: empty tiles sit at fixed row blocks, a CTA visits every 148th
// tile, and a height that shares a factor with 148 would hand some CTAs twice as many empty tiles as others.
constexpr int GROUP_M = 16, GROUP_M_COUNTS = 15;
__device__ __forceinline__ void tile_coords(int tile, int tiles_m, int tiles_n, int& m_blk, int& n_blk, int group_m = GROUP_M) {
  const int per_group = group_m * tiles_n;
  const int group = tile / per_group;
  const int first_m = group * group_m;
  const int gm = (tiles_m - first_m) < group_m ? (tiles_m - first_m) : group_m;
  const int in = tile - group * per_group;
  m_blk = first_m + in % gm;
  n_blk = in / gm;
}

template <bool A_MN, bool B_MN>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                 const GemmParams p) {
  extern __shared__ uint8_t smem_raw[];
  // operand stages need 1024-byte alignment for the 128-byte swizzle pattern
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
  uint64_t* full = bars;                  // [STAGES] TMA -> MMA
  uint64_t* empty = bars + STAGES;        // [STAGES] MMA -> TMA
  uint64_t* acc_full = bars + 2 * STAGES;   // [2] MMA -> epilogue
  uint64_t* acc_empty = bars + 2 * STAGES + 2;  // [2] epilogue -> MMA
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int tiles_per_problem = p.tiles_m * p.tiles_n;
  const int num_tiles = tiles_per_problem * p.batch;
  const int group_m = (p.counts != nullptr && !p.count_k) ? GROUP_M_COUNTS : GROUP_M;
  const int k_blocks = (p.K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&acc_full[b], 1);
      mbar_init(&acc_empty[b], 4);  // one arrival per epilogue warp
    }
    *abort_flag = 0;
    fence_barrier_init();
    tma_prefetch_desc(&map_a);
    tma_prefetch_desc(&map_b);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------- TMA producer --------------------------------------------
    // (all lanes walk the loop; one elected lane issues: see elect_one)
    {
      uint32_t it = 0;
      uint32_t armed = 0;       // bit s set <=> a copy into stage s may still be in flight
      uint32_t armed_phase = 0; // bit s = barrier phase of the latest copy issued into stage s
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        int m_blk, n_blk;
        const int prob = tile / tiles_per_problem;
        tile_coords(tile - prob * tiles_per_problem, p.tiles_m, p.tiles_n, m_blk, n_blk, group_m);
        const int m0 = m_blk * BM, n0 = n_blk * BN;
        const int a_row = prob * p.a_off, b_row = prob * p.b_off;  // storage-row offsets of this problem
        if (!tile_live(p, prob, m0)) continue;
        KRanges kr;
        int kb_lo, kb_hi;
        while (ok && kr.get(p, prob, k_blocks, kb_lo, kb_hi)) for (int kb = kb_lo; kb < kb_hi; ++kb) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!mbar_wait_bounded_warp(&empty[s], ph ^ 1, abort_flag, p.status)) { ok = false; break; }
          uint8_t* sa = smem + s * STAGE_BYTES;
          uint8_t* sb = sa + A_BYTES;
          armed |= 1u << s;
          armed_phase = (armed_phase & ~(1u << s)) | (ph << s);
          const int k0 = kb * BK;
          if (elect_one()) {
            mbar_expect_tx(&full[s], STAGE_BYTES);
            if (!A_MN) {
              tma_load_2d(sa, &map_a, &full[s], k0, a_row + m0);         // box {64 k, 128 rows}
            } else if (p.a_blocked) {
              tma_load_3d(sa, &map_a, &full[s], 0, a_row + k0, m0 >> 6); // box {64 m, 64 k, 2 blocks}
            } else {
#pragma unroll
              for (int j = 0; j < BM / 64; ++j) tma_load_2d(sa + j * 8192, &map_a, &full[s], m0 + j * 64, a_row + k0);
            }
            if (!B_MN) {
              tma_load_2d(sb, &map_b, &full[s], k0, b_row + n0);         // box {64 k, 256 rows}
            } else if (p.b_blocked) {
              tma_load_3d(sb, &map_b, &full[s], 0, b_row + k0, n0 >> 6); // box {64 n, 64 k, 4 blocks}
            } else {
#pragma unroll
              for (int j = 0; j < BN / 64; ++j) tma_load_2d(sb + j * 8192, &map_b, &full[s], n0 + j * 64, b_row + k0);
            }
          }
          __syncwarp();
          ++it;
        }
      }
      if (!ok) {
        // drain: wait (bounded) until every copy this thread issued has landed, so that no TMA write is
        // still in flight when the CTA's shared memory is released
        const uint64_t t0 = globaltimer_ns();
        for (int s = 0; s < STAGES; ++s) {
          if (!(armed & (1u << s))) continue;
          const uint32_t ph = (armed_phase >> s) & 1;
          while (!mbar_try_wait(&full[s], ph) && globaltimer_ns() - t0 < wait_budget_ns()) {
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------- MMA issuer --------------------------------------------------
    {
      constexpr uint32_t idesc = make_idesc_bf16(BM, BN, A_MN, B_MN);
      uint32_t it = 0;
      uint32_t tile_i = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        const int prob = tile / tiles_per_problem;
        if (p.counts != nullptr) {
          int m_blk, n_blk;
          tile_coords(tile - prob * tiles_per_problem, p.tiles_m, p.tiles_n, m_blk, n_blk, group_m);
          if (!tile_live(p, prob, m_blk * BM)) continue;
        }
        const uint32_t acc = tile_i & 1;
        const uint32_t acc_ph = (tile_i >> 1) & 1;
        if (!mbar_wait_bounded_warp(&acc_empty[acc], acc_ph ^ 1, abort_flag, p.status)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        bool fresh = true;  // the first product of a tile overwrites the accumulator
        KRanges kr;
        int kb_lo, kb_hi;
        while (ok && kr.get(p, prob, k_blocks, kb_lo, kb_hi)) for (int kb = kb_lo; kb < kb_hi; ++kb) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!mbar_wait_bounded_warp(&full[s], ph, abort_flag, p.status)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + s * STAGE_BYTES);
          const uint32_t sb = sa + A_BYTES;
          if (elect_one()) {
#pragma unroll
            for (int k = 0; k < BK / UMMA_K; ++k) {
              const uint64_t da = A_MN ? make_smem_desc(sa + k * 2048, 8192, 1024) : make_smem_desc(sa + k * 32, 16, 1024);
              const uint64_t db = B_MN ? make_smem_desc(sb + k * 2048, 8192, 1024) : make_smem_desc(sb + k * 32, 16, 1024);
              umma_bf16_ss(d_tmem, da, db, idesc, !(fresh && k == 0));
            }
            umma_commit(&empty[s]);  // frees the stage once these MMAs have read it
          }
          __syncwarp();
          fresh = false;
          ++it;
        }
        if (ok && elect_one()) umma_commit(&acc_full[acc]);
        __syncwarp();
        ++tile_i;
      }
    }
  } else {
    // ------------------------------- epilogue (warps 2..5) ------------------------------------------
    const int quarter = warp & 3;  // TMEM lanes [32*quarter, 32*quarter+32) are visible to this warp
    uint32_t tile_i = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
      int m_blk, n_blk;
      const int prob = tile / tiles_per_problem;
      tile_coords(tile - prob * tiles_per_problem, p.tiles_m, p.tiles_n, m_blk, n_blk, group_m);
      const int m0 = m_blk * BM, n0 = n_blk * BN;
      if (!tile_live(p, prob, m0)) {  // uniform across the CTA: nothing was computed, the tile is all zeros
        if (p.accumulate) continue;   // nothing to add
        const int row_z = m0 + quarter * 32;   // this warp's 32 rows, one row at a time, lanes along the columns
        const int n_end = min(n0 + BN, p.N);
        for (int rr = 0; rr < 32 && row_z + rr < p.M; ++rr) {
          const size_t row = size_t(prob) * p.M + row_z + rr;
          if (p.out_fp32) {
            float* d = static_cast<float*>(p.D) + row * p.ldd;
            for (int c = n0 + lane; c < n_end; c += 32) d[c] = 0.f;
          } else {
            __nv_bfloat16* d = static_cast<__nv_bfloat16*>(p.D) + row * p.ldd;
            for (int c = n0 + lane; c < n_end; c += 32) d[c] = __float2bfloat16_rn(0.f);
          }
        }
        continue;
      }
      const uint32_t acc = tile_i & 1;
      const uint32_t acc_ph = (tile_i >> 1) & 1;
      if (!mbar_wait_bounded_warp(&acc_full[acc], acc_ph, abort_flag, p.status)) { ok = false; break; }
      tc_fence_after();
      const int row_in = m0 + quarter * 32 + lane;        // row within this problem
      const bool row_ok = row_in < p.M;
      const size_t row = size_t(prob) * p.M + row_in;     // row of the stacked output
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        const int col0 = n0 + c * 32;
        if (col0 >= p.N) break;  // uniform across the warp
        uint32_t r[32];
        tmem_ld_32x32(tmem_base + (uint32_t(quarter * 32) << 16) + acc * BN + c * 32, r);
        tc_wait_ld();
        float v[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
        if (p.bias) {
          if (p.bias_fp32) {
            const float* b = static_cast<const float*>(p.bias) + col0;
#pragma unroll
            for (int j = 0; j < 32; ++j) if (col0 + j < p.N) v[j] += __ldg(b + j);
          } else {
            const __nv_bfloat16* b = static_cast<const __nv_bfloat16*>(p.bias) + col0;
#pragma unroll
            for (int j = 0; j < 32; ++j) if (col0 + j < p.N) v[j] += __bfloat162float(b[j]);
          }
        }
        if (!row_ok) continue;
        const bool full_chunk = col0 + 32 <= p.N;
        if (p.out_fp32) {
          float* d = static_cast<float*>(p.D) + row * p.ldd + col0;
          if (full_chunk && (p.ldd & 3) == 0) {
#pragma unroll
            for (int j = 0; j < 32; j += 4) {
              float4 o = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
              if (p.accumulate) {
                const float4 old = *reinterpret_cast<const float4*>(d + j);
                o.x += old.x; o.y += old.y; o.z += old.z; o.w += old.w;
              }
              *reinterpret_cast<float4*>(d + j) = o;
            }
          } else {
            for (int j = 0; j < 32 && col0 + j < p.N; ++j) d[j] = p.accumulate ? d[j] + v[j] : v[j];
          }
        } else {
          __nv_bfloat16* d = static_cast<__nv_bfloat16*>(p.D) + row * p.ldd + col0;
          if (full_chunk && (p.ldd & 7) == 0) {
#pragma unroll
            for (int j = 0; j < 32; j += 8) {
              uint4 o;
              o.x = pack_bf16(v[j], v[j + 1]);
              o.y = pack_bf16(v[j + 2], v[j + 3]);
              o.z = pack_bf16(v[j + 4], v[j + 5]);
              o.w = pack_bf16(v[j + 6], v[j + 7]);
              *reinterpret_cast<uint4*>(d + j) = o;
            }
          } else {
            for (int j = 0; j < 32 && col0 + j < p.N; ++j) d[j] = __float2bfloat16_rn(v[j]);
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[acc]);
      ++tile_i;
    }
  }

  // ------------------------------- teardown -------------------------------------------------------------
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// -------------------------------------------------------------------------------------------------------------
// host side: tensor-map cache + launcher
// -------------------------------------------------------------------------------------------------------------
struct MapKey {
  const void* base;
  uint64_t d0, d1, stride;
  uint32_t b0, b1;
  bool operator==(const MapKey& o) const {
    return base == o.base && d0 == o.d0 && d1 == o.d1 && stride == o.stride && b0 == o.b0 && b1 == o.b1;
  }
};
struct MapKeyHash {
  size_t operator()(const MapKey& k) const {
    size_t h = reinterpret_cast<size_t>(k.base);
    h = h * 1000003u ^ k.d0;
    h = h * 1000003u ^ k.d1;
    h = h * 1000003u ^ k.stride;
    h = h * 1000003u ^ (size_t(k.b0) << 16 | k.b1);
    return h;
  }
};

static std::mutex g_map_mutex;
static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> g_map_cache;

// 2-D bf16 map over a row-major matrix with `rows` rows of `cols` contiguous elements.
static int get_map_2d(CUtensorMap* out, const void* base, uint64_t cols, uint64_t rows, uint64_t ld_elems,
                      uint32_t box_cols, uint32_t box_rows) {
  MapKey key{base, cols, rows, ld_elems, box_cols, box_rows};
  {
    std::lock_guard<std::mutex> lock(g_map_mutex);
    auto it = g_map_cache.find(key);
    if (it != g_map_cache.end()) {
      *out = it->second;
      return 0;
    }
  }
  uint64_t dims[2] = {cols, rows};
  uint64_t strides[1] = {ld_elems * 2};
  uint32_t box[2] = {box_cols, box_rows};
  int rc = jpb_make_tensor_map(out, base, 2, 2, dims, strides, box, 1);
  if (rc != 0) return rc;
  std::lock_guard<std::mutex> lock(g_map_mutex);
  if (g_map_cache.size() > 4096) g_map_cache.clear();
  g_map_cache.emplace(key, *out);
  return 0;
}

// 3-D bf16 map over an MN-major operand stored as [K rows, mn contiguous] (mn a multiple of 64): dimensions
// {64 within a block, K, mn / 64 blocks}; one copy of box {64, 64, blocks} lands as `blocks` consecutive
// 64x64 swizzled blocks, the layout the MN-major shared-memory descriptors expect.
static int get_map_mn_blocked(CUtensorMap* out, const void* base, uint64_t mn, uint64_t k_rows, uint64_t ld_elems,
                              uint32_t blocks) {
  MapKey key{base, mn, k_rows, ld_elems, 0xB10Cu, blocks};
  {
    std::lock_guard<std::mutex> lock(g_map_mutex);
    auto it = g_map_cache.find(key);
    if (it != g_map_cache.end()) {
      *out = it->second;
      return 0;
    }
  }
  uint64_t dims[3] = {64, k_rows, mn / 64};
  uint64_t strides[2] = {ld_elems * 2, 128};
  uint32_t box[3] = {64, 64, blocks};
  int rc = jpb_make_tensor_map(out, base, 2, 3, dims, strides, box, 1);
  if (rc != 0) return rc;
  std::lock_guard<std::mutex> lock(g_map_mutex);
  if (g_map_cache.size() > 4096) g_map_cache.clear();
  g_map_cache.emplace(key, *out);
  return 0;
}

static int g_num_sms = 0;

template <bool A_MN, bool B_MN>
static int launch(const CUtensorMap& ma, const CUtensorMap& mb, const GemmParams& p, cudaStream_t stream) {
  auto kernel = gemm_bf16_kernel<A_MN, B_MN>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    if (e != cudaSuccess) return int(e);
    configured = true;
  }
  if (g_num_sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&g_num_sms, cudaDevAttrMultiProcessorCount, dev);
  }
  const int tiles = p.tiles_m * p.tiles_n * p.batch;
  const int grid = tiles < g_num_sms ? tiles : g_num_sms;
  kernel<<<grid, GEMM_THREADS, SMEM_BYTES, stream>>>(ma, mb, p);
  return int(cudaGetLastError());
}

}  // namespace jpb

// Common entry: `batch` equal-sized problems stacked along the storage rows of A, B and D (batch == 1: one GEMM).
static int gemm_entry(const void* A, const void* B, void* D, const void* bias, int batch, int M, int N, int K, int lda, int ldb,
                      int ldd, int a_mn_major, int b_mn_major, int out_fp32, int accumulate, int bias_fp32, void* stream,
                      const int* counts = nullptr, int seg_rows = 0, int segs = 0, int count_k = 0) {
  using namespace jpb;
  if (M <= 0 || N <= 0 || K <= 0 || batch <= 0) return 0;
  if (counts != nullptr) {
    // segments must tile the counted dimension exactly; a bias would make dead tiles non-zero
    if (seg_rows <= 0 || segs <= 0 || (long long)seg_rows * segs != (count_k ? K : M) || bias != nullptr || K % BK != 0)
      return -JPB_ERR_BAD_ARGUMENT;
  }
  if ((reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15) || (lda & 7) || (ldb & 7))
    return -JPB_ERR_BAD_ARGUMENT;
  if (accumulate && !out_fp32) return -JPB_ERR_BAD_ARGUMENT;
  if (batch > 1 && (K % BK != 0 || bias != nullptr)) return -JPB_ERR_BAD_ARGUMENT;
  CUtensorMap ma, mb;
  int rc;
  const uint64_t nb = uint64_t(batch);
  const int a_blocked = a_mn_major && M % 64 == 0, b_blocked = b_mn_major && N % 64 == 0;
  if (!a_mn_major) rc = get_map_2d(&ma, A, K, nb * M, lda, BK, BM);
  else if (a_blocked) rc = get_map_mn_blocked(&ma, A, M, nb * K, lda, BM / 64);
  else rc = get_map_2d(&ma, A, M, nb * K, lda, 64, BK);
  if (rc) return rc;
  if (!b_mn_major) rc = get_map_2d(&mb, B, K, nb * N, ldb, BK, BN);
  else if (b_blocked) rc = get_map_mn_blocked(&mb, B, N, nb * K, ldb, BN / 64);
  else rc = get_map_2d(&mb, B, N, nb * K, ldb, 64, BK);
  if (rc) return rc;
  GemmParams p;
  p.a_blocked = a_blocked; p.b_blocked = b_blocked;
  p.batch = batch;
  p.a_off = a_mn_major ? K : M;
  p.b_off = b_mn_major ? K : N;
  p.M = M; p.N = N; p.K = K; p.ldd = ldd; p.out_fp32 = out_fp32; p.accumulate = accumulate;
  p.bias = bias; p.bias_fp32 = bias_fp32; p.D = D; p.status = jpb_status_device_ptr();
  p.tiles_m = (M + BM - 1) / BM;
  p.tiles_n = (N + BN - 1) / BN;
  p.counts = counts; p.seg_rows = seg_rows; p.segs = segs; p.count_k = count_k;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (!a_mn_major && !b_mn_major) return launch<false, false>(ma, mb, p, s);
  if (!a_mn_major && b_mn_major) return launch<false, true>(ma, mb, p, s);
  if (a_mn_major && b_mn_major) return launch<true, true>(ma, mb, p, s);
  return launch<true, false>(ma, mb, p, s);
}

// A: [M,K] with lda (K-major) or stored as [K,M] with lda (MN-major); likewise B for [N,K] / [K,N].
// All leading dimensions in elements; bf16 operands must be 16-byte aligned with lda/ldb multiples of 8.
JPB_API int jpb_gemm_bf16(const void* A, const void* B, void* D, const void* bias, int M, int N, int K, int lda, int ldb,
                          int ldd, int a_mn_major, int b_mn_major, int out_fp32, int accumulate, int bias_fp32,
                          void* stream) {
  return gemm_entry(A, B, D, bias, 1, M, N, K, lda, ldb, ldd, a_mn_major, b_mn_major, out_fp32, accumulate, bias_fp32, stream);
}

// Grouped GEMM with equal-sized groups (the local experts of a mixture-of-experts layer): problem b uses rows
// [b*M, (b+1)*M) of a K-major A (or rows [b*K, (b+1)*K) of an MN-major one), likewise B, and writes rows
// [b*M, (b+1)*M) of D.  One launch, one persistent grid over all problems' tiles.  K must be a multiple of 64.
JPB_API int jpb_gemm_bf16_batched(const void* A, const void* B, void* D, int batch, int M, int N, int K, int lda, int ldb,
                                  int ldd, int a_mn_major, int b_mn_major, int out_fp32, int accumulate, void* stream) {
  return gemm_entry(A, B, D, nullptr, batch, M, N, K, lda, ldb, ldd, a_mn_major, b_mn_major, out_fp32, accumulate, 0, stream);
}

// Grouped GEMM whose groups differ in size (a mixture-of-experts layer after capacity routing: every expert has room
// for the same number of slots, but fills only some).  Storage is that of jpb_gemm_bf16_batched; `counts` (device
// memory, [batch, segs] int32) says how many rows at the start of each `seg_rows`-row segment hold data -- segments of
// the M rows of each problem (count_k = 0: forward and input gradient), or of its K reduction rows (count_k = 1:
// weight gradient).  The other rows must be zero.  Output tiles and 64-row reduction blocks without a live row cost no
// memory traffic and no tensor-core time; the result equals that of jpb_gemm_bf16_batched.
JPB_API int jpb_gemm_bf16_grouped(const void* A, const void* B, void* D, int batch, int M, int N, int K, int lda, int ldb,
                                  int ldd, int a_mn_major, int b_mn_major, int out_fp32, int accumulate, const int* counts,
                                  int seg_rows, int segs, int count_k, void* stream) {
  if (counts == nullptr) return -JPB_ERR_BAD_ARGUMENT;
  return gemm_entry(A, B, D, nullptr, batch, M, N, K, lda, ldb, ldd, a_mn_major, b_mn_major, out_fp32, accumulate, 0, stream,
                    counts, seg_rows, segs, count_k);
}
