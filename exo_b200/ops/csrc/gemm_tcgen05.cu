// bf16 GEMM on the 5th-generation tensor cores:  out[M, N] = x[M, K] . W[N, K]^T  (+bias)(+residual).
//
// The problem is issued "swapped": the weight tile is the MMA's M operand (128 output features on
// the 128 TMEM lanes) and the activation rows are the MMA's N operand (BN = 16..256 columns).  Both
// operands are K-major in memory as they are, so no transpose is ever materialised, and a decode
// batch of 9..256 rows maps onto ONE instruction shape without padding the batch to 128.  The
// kernel is therefore weight-bandwidth bound for decode and tensor bound for prefill.
//
// CTA = 6 warps:  warp 0 = TMA producer (one elected lane), warp 1 = TMEM owner + MMA issuer (one
// elected lane), warps 2..5 = epilogue (tcgen05.ld of the four 32-lane TMEM quadrants).
// Pipeline: STAGES x {W tile 128x64, x tile BNx64} in 128B-swizzled shared memory, full/empty
// mbarriers, accumulator in TMEM, tcgen05.commit releases stages and publishes the accumulator.
//
// Split-K (grid.z): each split writes an fp32 partial tile to a workspace; the last CTA to arrive
// on the tile's counter sums the partials in split order (deterministic) and runs the epilogue.
#include <mutex>
#include <unordered_map>

#include <cstdlib>
#include <cstring>
#include "gemm_common.cuh"
#include "status.h"

namespace {

using gemm::BM;
using gemm::BK;
using gemm::GemmParams;

// TWO: the CTA owns two 128-feature weight tiles (two accumulators) that share every activation
// tile, so a [256 x 256] output block costs 64 KB of shared-memory traffic per K step instead of
// 96 KB — the prefill shapes are bound by the L2 -> SM path, not by the tensor pipe.
template <int BN, int STAGES, bool TWO>
struct Smem {
  alignas(1024) __nv_bfloat16 a[STAGES][(TWO ? 2 : 1) * BM * BK];
  alignas(1024) __nv_bfloat16 b[STAGES][BN * BK];
  uint64_t full[STAGES], empty[STAGES], acc_full;
  uint32_t tmem_base;
  int abort_flag;
  int is_last;
};

// GLU (with TWO): the two weight tiles are the gate rows and the up rows of the same 128 features of a fused
// [gate; up] matrix and the epilogue writes silu(gate) * up — the SwiGLU kernel and its traffic disappear.
template <int BN, int STAGES, bool TWO, bool HO, bool GLU = false>
__global__ void __launch_bounds__(192, (BN <= 128 ? 2 : 1))
gemm_swapped_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_x,
                    const GemmParams p) {
  extern __shared__ uint8_t smem_raw[];
  using S = Smem<BN, STAGES, TWO>;
  S& s = *reinterpret_cast<S*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  constexpr uint32_t TMEM_COLS = (TWO ? 2 : 1) * BN < 32 ? 32 : (TWO ? 2 : 1) * BN;
  // the prefill kernels (BN = 256) may run with fewer activation rows per CTA than BN, so that the tile count fits
  // whole waves over the SMs: the accumulators keep their BN-column spacing, the MMAs and the epilogue are bn wide
  const int bn = p.bn_rows > 0 ? p.bn_rows : BN;
  const uint32_t STAGE_BYTES = ((TWO ? 2 : 1) * BM * BK + bn * BK) * 2;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // Prefill launches walk the row tiles fastest: the CTAs that run together then share a few weight tiles (each read
  // from HBM once) and re-read the activations, which are the smaller operand and stay in L2; with the feature tiles
  // fastest every wave streamed a different set of weight tiles and a matrix larger than L2 was re-read once per row tile.
  const unsigned tile_n = p.rows_fastest ? blockIdx.y : blockIdx.x, tile_m = p.rows_fastest ? blockIdx.x : blockIdx.y;
  const unsigned tiles_m = p.rows_fastest ? gridDim.x : gridDim.y;
  const int n0 = (int)tile_n * BM * ((TWO && !GLU) ? 2 : 1), split = blockIdx.z;
  const int m0 = (int)((tile_m + (unsigned)p.m_tile_shift) % tiles_m) * bn;
  const int second = GLU ? p.N / 2 : BM;      // row distance of the second weight tile
  const int kb_total = (p.K + BK - 1) / BK;
  const int kb0 = split * p.kb_per_split;
  const int nkb = min(p.kb_per_split, kb_total - kb0);

  if (threadIdx.x == 0) {
    for (int i = 0; i < STAGES; i++) { tc::mbar_init(&s.full[i], 1); tc::mbar_init(&s.empty[i], 1); }
    tc::mbar_init(&s.acc_full, 1);
    s.abort_flag = 0;
    s.is_last = 0;
    tc::fence_barrier_init();
  }
  if (warp == 1) {
    tc::tmem_alloc(&s.tmem_base, TMEM_COLS);
    tc::tmem_relinquish();
  }
  tc::tc_fence_before();
  __syncthreads();
  tc::tc_fence_after();
  const uint32_t tmem = s.tmem_base;

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (tc::elect_one()) {
      tc::prefetch_tmap(&tmap_w);
      tc::prefetch_tmap(&tmap_x);
      bool gate_ok = true;
      if (p.row_flags) {
        // all-gather -> GEMM: this CTA's activation rows belong to one or two ranks; wait (bounded) until those ranks
        // have delivered them, then order the wait before the TMA engine's reads of the same memory
        const int o_lo = m0 / p.rows_per_flag, o_hi = (min(p.M, m0 + bn) - 1) / p.rows_per_flag;
        unsigned long long t0;
        asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t0));
        const int need = *reinterpret_cast<const volatile int*>(p.row_epoch);
        for (int o = o_lo; o <= o_hi && gate_ok; o++) {
          while (tp_ld_acquire_sys(p.row_flags + o) - need < 0) {
            unsigned long long now;
            asm volatile("mov.u64 %0, %globaltimer;" : "=l"(now));
            if (now - t0 > p.gate_wait_ns) {
              atomicExch(p.gate_status, 4 /* peer timeout */);
              s.abort_flag = 1;
              gate_ok = false;
              break;
            }
            __nanosleep(64);
          }
        }
        asm volatile("fence.proxy.async;" ::: "memory");
      }
      for (int i = 0; i < nkb && gate_ok; i++) {
        int st = i % STAGES;
        if (i >= STAGES && !tc::mbar_wait(&s.empty[st], ((i / STAGES) - 1) & 1)) {
          atomicExch(p.err, tc::ERR_EMPTY_TIMEOUT);
          s.abort_flag = 1;
          break;
        }
        tc::mbar_expect_tx(&s.full[st], STAGE_BYTES);
        int k = (kb0 + i) * BK;
        tc::tma_load_2d(s.a[st], &tmap_w, k, n0, &s.full[st]);
        if constexpr (TWO) tc::tma_load_2d(s.a[st] + BM * BK, &tmap_w, k, n0 + second, &s.full[st]);
        tc::tma_load_2d(s.b[st], &tmap_x, k, m0, &s.full[st]);
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer ------------------------------
    if (tc::elect_one()) {
      const uint32_t idesc = tc::umma_idesc_bf16(BM, bn);
      bool ok = true;
      for (int i = 0; i < nkb && ok; i++) {
        int st = i % STAGES;
        if (!tc::mbar_wait(&s.full[st], (i / STAGES) & 1)) {
          atomicExch(p.err, tc::ERR_FULL_TIMEOUT);
          s.abort_flag = 1;
          ok = false;
          break;
        }
        tc::tc_fence_after();
        uint64_t ad = tc::umma_desc_sw128(tc::smem_u32(s.a[st]));
        uint64_t bd = tc::umma_desc_sw128(tc::smem_u32(s.b[st]));
#pragma unroll
        for (int k = 0; k < BK / 16; k++) {  // +32 bytes per K step of 16 bf16 → +2 in the >>4 address field
          tc::umma_bf16(tmem, ad + 2 * k, bd + 2 * k, idesc, (i | k) != 0);
          if constexpr (TWO) {
            const uint64_t ad2 = tc::umma_desc_sw128(tc::smem_u32(s.a[st] + BM * BK));
            tc::umma_bf16(tmem + BN, ad2 + 2 * k, bd + 2 * k, idesc, (i | k) != 0);
          }
        }
        tc::umma_commit(&s.empty[st]);  // stage reusable once these MMAs have read it
      }
      tc::umma_commit(&s.acc_full);  // accumulator complete (also arrives if we bailed out: nothing pending)
    }
  } else {
    if constexpr (GLU) {
      gemm::epilogue_swiglu<BN>(p, tmem, &s.acc_full, &s.abort_flag, n0, m0, nkb, warp, lane, bn);
    } else {
    gemm::epilogue<BN, HO>(p, tmem, &s.acc_full, &s.abort_flag, &s.is_last, n0, m0, split, nkb, warp, lane, bn);
    // second accumulator: plain stores only (the launcher uses TWO without split-K or hand-over)
    if constexpr (TWO) gemm::epilogue<BN>(p, tmem + BN, &s.acc_full, &s.abort_flag, &s.is_last, n0 + BM, m0, split, nkb, warp, lane, bn);
    }
  }
  // ------------------------------ teardown ------------------------------
  tc::tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc::tc_fence_after();
    tc::tmem_dealloc(tmem, TMEM_COLS);
  }
}

// ------------------------------------------------------------------------------------------
// host side
// ------------------------------------------------------------------------------------------
typedef CUresult (*EncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                             const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                             CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeFn get_encode() {
  static EncodeFn fn = nullptr;
  static bool tried = false;
  if (!tried) {
    tried = true;
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = (EncodeFn)p;
  }
  return fn;
}

struct Key {
  const void* base; uint64_t rows, cols; uint32_t box;   // box: rows of the box, | 1<<31 for the byte-typed maps
  bool operator==(const Key& o) const { return base == o.base && rows == o.rows && cols == o.cols && box == o.box; }
};
struct KeyHash {
  size_t operator()(const Key& k) const {
    return std::hash<uint64_t>()((uint64_t)k.base * 1000003u ^ k.rows * 7919u ^ k.cols * 104729u ^ k.box);
  }
};
std::unordered_map<Key, CUtensorMap, KeyHash> g_maps;   // descriptors by value: eviction never frees what a caller holds
std::mutex g_maps_mu;

// Lookups hand out a COPY of the cached descriptor in a per-thread ring.  A launcher fetches a handful of maps
// (weights, activations, K, V ...) and then launches, so a pointer stays valid for the next RING - 1 lookups of the
// same thread whatever happens to the cache in between (another thread's insert may evict everything).
constexpr int TMAP_RING = 32;
const CUtensorMap* ring_copy(const CUtensorMap& m) {
  thread_local CUtensorMap ring[TMAP_RING];
  thread_local int next = 0;
  CUtensorMap* slot = &ring[next];
  next = (next + 1) % TMAP_RING;
  *slot = m;
  return slot;
}

int* g_err[16] = {nullptr};
int* g_counters[16] = {nullptr};
float* g_partial[16] = {nullptr};
size_t g_partial_floats[16] = {0};
constexpr int MAX_TILES = 1 << 16;
constexpr size_t MAX_CACHED_MAPS = 8192;

const CUtensorMap* tmap_lookup(const void* base, uint64_t rows, uint64_t cols, uint32_t box_rows, bool bytes) {
  std::lock_guard<std::mutex> lk(g_maps_mu);
  Key k{base, rows, cols, box_rows | (bytes ? (1u << 31) : 0u)};
  auto it = g_maps.find(k);
  if (it != g_maps.end()) return ring_copy(it->second);
  EncodeFn enc = get_encode();
  const uint64_t el = bytes ? 1 : 2;
  if (!enc || (cols * el) % 16 != 0 || ((uintptr_t)base & 15)) return nullptr;
  CUtensorMap m;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {cols * el};
  cuuint32_t box[2] = {(cuuint32_t)BK, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(&m, bytes ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base),
                   dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   bytes ? CU_TENSOR_MAP_SWIZZLE_NONE : CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return nullptr;
  if (g_maps.size() >= MAX_CACHED_MAPS) g_maps.clear();  // activations come and go: bound the cache (re-encoding is cheap)
  g_maps[k] = m;
  return ring_copy(m);
}

}  // namespace

// K-major bf16 [rows, cols] matrix, [box_rows x 64] box, 128-byte swizzle.  The returned pointer addresses a
// per-thread copy that stays valid for the next 31 lookups made by the calling thread.
const CUtensorMap* exo_tmap_2d_bf16(const void* base, uint64_t rows, uint64_t cols, uint32_t box_rows) {
  return tmap_lookup(base, rows, cols, box_rows, false);
}

// Row-major [rows, cols] byte matrix (fp8 payloads) with a [box_rows x 64] box, no swizzle: the
// consumer reads the tile with ordinary shared-memory loads.  Same pointer lifetime as above.
const CUtensorMap* exo_tmap_2d_u8(const void* base, uint64_t rows, uint64_t cols, uint32_t box_rows) {
  return tmap_lookup(base, rows, cols, box_rows, true);
}

// The current device's scratch of the GEMM family (null / 0 before exo_gemm_init).
int exo_gemm_scratch(int** err, int** counters, float** partial, size_t* partial_floats) {
  int dev;
  if (cudaGetDevice(&dev) != cudaSuccess || dev >= 16 || !g_err[dev]) return -4;
  *err = g_err[dev];
  *counters = g_counters[dev];
  *partial = g_partial[dev];
  *partial_floats = g_partial_floats[dev];
  return 0;
}

// Per-device scratch set up on first use (NOT inside stream capture: call exo_gemm_init first).
EXO_API int exo_gemm_init(long partial_floats) {
  int dev;
  if (cudaGetDevice(&dev) != cudaSuccess || dev >= 16) return -1;
  if (!g_err[dev]) {
    g_err[dev] = exo_status_word(EXO_STATUS_TC);      // host-mapped status word: the serving loop reads it without a copy
    if (!g_err[dev]) return -1;
    if (cudaMalloc(&g_counters[dev], MAX_TILES * sizeof(int)) != cudaSuccess) return -1;
    cudaMemset(g_counters[dev], 0, MAX_TILES * sizeof(int));
  }
  if ((size_t)partial_floats > g_partial_floats[dev]) {
    if (g_partial[dev]) cudaFree(g_partial[dev]);
    if (cudaMalloc(&g_partial[dev], (size_t)partial_floats * sizeof(float)) != cudaSuccess) return -1;
    g_partial_floats[dev] = (size_t)partial_floats;
  }
  return 0;
}

// The device error word of the current device, shared by every tensor-core kernel (nullptr before exo_gemm_init).
int* exo_tc_err_ptr() {
  int dev;
  if (cudaGetDevice(&dev) != cudaSuccess || dev >= 16) return nullptr;
  return g_err[dev];
}

// Reads and clears the tensor-core kernels' status word (no device access; call once the kernels have completed).
EXO_API int exo_gemm_last_error() { return exo_status_take(EXO_STATUS_TC, 1); }

template <int BN, int STAGES, bool TWO = false, bool HO = false>
static int launch_gemm_ho(const CUtensorMap* tw, const CUtensorMap* tx, const GemmParams& p, cudaStream_t st) {
  using S = Smem<BN, STAGES, TWO>;
  size_t smem = sizeof(S) + 1024;
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(gemm_swapped_kernel<BN, STAGES, TWO, HO>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) !=
        cudaSuccess)
      return -3;
    attr_set = true;
  }
  constexpr int FEATS = BM * (TWO ? 2 : 1);
  const int bn = p.bn_rows > 0 ? p.bn_rows : BN;
  dim3 grid((p.N + FEATS - 1) / FEATS, (p.M + bn - 1) / bn, p.splits);
  if (p.rows_fastest) grid = dim3(grid.y, grid.x, 1);
  gemm_swapped_kernel<BN, STAGES, TWO, HO><<<grid, 192, smem, st>>>(*tw, *tx, p);
  EXO_CHECK_LAUNCH();
  return 0;
}

static int launch_gemm_glu(const CUtensorMap* tw, const CUtensorMap* tx, const GemmParams& p, cudaStream_t st) {
  using S = Smem<256, 3, true>;
  const size_t smem = sizeof(S) + 1024;
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(gemm_swapped_kernel<256, 3, true, false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             (int)smem) != cudaSuccess)
      return -3;
    attr_set = true;
  }
  const int bn = p.bn_rows > 0 ? p.bn_rows : 256;
  dim3 grid((p.N / 2 + BM - 1) / BM, (p.M + bn - 1) / bn, 1);
  if (p.rows_fastest) grid = dim3(grid.y, grid.x, 1);
  gemm_swapped_kernel<256, 3, true, false, true><<<grid, 192, smem, st>>>(*tw, *tx, p);
  EXO_CHECK_LAUNCH();
  return 0;
}

template <int BN, int STAGES, bool TWO = false>
static int launch_gemm(const CUtensorMap* tw, const CUtensorMap* tx, const GemmParams& p, cudaStream_t st) {
  if constexpr (!TWO) {
    if (p.ho.n_ll > 0) return launch_gemm_ho<BN, STAGES, false, true>(tw, tx, p, st);
  }
  return launch_gemm_ho<BN, STAGES, TWO, false>(tw, tx, p, st);
}

// Activation rows per CTA of a prefill launch with `tiles_n` feature tiles: the multiple of 16 in [128, 256] that
// minimises  waves x (rows + fixed)  over the 148 SMs, where `fixed` stands for a tile's prologue and epilogue (about
// 15 % of a full tile's main loop).  Returns the rows and, in *cost, that product (for comparing tile shapes).
// Example: two-accumulator tiles, N = 6144 (24 feature tiles), M = 2048: 256 rows is 192 CTAs = two waves, the second
// 30 % full; 176 rows is 288 CTAs = two waves of 0.69-size tiles.
static int fit_rows(long tiles_n, int M, long* cost_out = nullptr) {
  static const bool off = getenv("EXO_GEMM_FIXED_ROWS") != nullptr;      // A/B switch, read once
  int best = 256;
  long best_cost = -1;
  for (int bn = 256; bn >= (off ? 256 : 128); bn -= 16) {
    const long ctas = tiles_n * ((M + bn - 1) / bn);
    const long cost = ((ctas + 147) / 148) * (bn + 38);
    if (best_cost < 0 || cost < best_cost) { best = bn; best_cost = cost; }
  }
  if (cost_out) *cost_out = best_cost;
  return best;
}

static int rows_fastest_default() {
  static const int v = getenv("EXO_GEMM_FEATURES_FASTEST") ? 0 : 1;      // A/B switch, read once
  return v;
}

// Suggested split count for a (M, N, K) problem: fill the 148 SMs when there are few output tiles.
EXO_API int exo_gemm_splits(int M, int N, int K) {
  int bn = M <= 16 ? 16 : M <= 32 ? 32 : M <= 64 ? 64 : M <= 128 ? 128 : 256;
  long tiles = (long)((N + BM - 1) / BM) * ((M + bn - 1) / bn);
  int kb = (K + BK - 1) / BK;
  // two CTAs are co-resident per SM (BN <= 128): aim for ~296 CTAs so every SM streams weights
  int target = bn <= 128 ? 296 : 148;
  if (M > 64) return 1;  // tensor-bound shapes: a split only adds a reduction pass
  if (tiles * 4 >= target * 3 || kb < 8) return 1;
  int s = (int)((target + tiles / 2) / tiles);
  if (s > kb / 4) s = kb / 4;
  if (s > 16) s = 16;
  return s < 1 ? 1 : s;
}

static int gemm_launch(const void* x, const void* W, const void* bias, const void* residual, void* out, int M, int N,
                       int K, int ldo, int splits, const TpHandover* ho, cudaStream_t st);

EXO_API int exo_gemm_bf16(const void* x, const void* W, const void* bias, const void* residual, void* out, int M, int N,
                          int K, int ldo, int splits, cudaStream_t st) {
  return gemm_launch(x, W, bias, residual, out, M, N, K, ldo, splits, nullptr, st);
}

int exo_comm_gate(int parity, int rows, const int** flags, const int** epoch, int* rows_per_flag, int* rank,
                  unsigned long long* wait_ns, int** status);

// Fills the all-gather -> GEMM fields of `p`: the rows of `x` are the broadcast output of the deferred-wait two-shot
// reduction on `parity` (see comm.cu); the row tiles are walked starting at this rank's own rows.
static int gate_params(GemmParams* p, int parity, int M, int bn) {
  int rank = 0;
  int rc = exo_comm_gate(parity, M, &p->row_flags, &p->row_epoch, &p->rows_per_flag, &rank, &p->gate_wait_ns, &p->gate_status);
  if (rc) return rc;
  p->m_tile_shift = (rank * p->rows_per_flag) / bn;
  return 0;
}

static int g_gate_parity = -1;      // >= 0: the next GEMM launched from this thread is gated on that parity

// All-gather -> GEMM: like exo_gemm_bf16 (M >= 256, no split-K), with the activation rows arriving from the other
// ranks while the kernel runs.
EXO_API int exo_gemm_bf16_gated(const void* x, const void* W, const void* bias, const void* residual, void* out, int M, int N,
                                int K, int ldo, int parity, cudaStream_t st) {
  if (M < 256) return -2;
  g_gate_parity = parity;
  int rc = gemm_launch(x, W, bias, residual, out, M, N, K, ldo, 1, nullptr, st);
  g_gate_parity = -1;
  return rc;
}

// Fused gate/up projection with the SwiGLU in the epilogue: W = [gate (F rows); up (F rows)], out[M, F].
// Prefill shapes only (M >= 256, no bias): returns -2 otherwise and the caller takes the two-kernel form.
static int gemm_swiglu_launch(const void* x, const void* W, void* out, int M, int N, int K, int gate_parity, cudaStream_t st);

EXO_API int exo_gemm_bf16_swiglu(const void* x, const void* W, void* out, int M, int N, int K, cudaStream_t st) {
  return gemm_swiglu_launch(x, W, out, M, N, K, -1, st);
}

// The same with the activation rows gated on the deferred-wait two-shot reduction of `parity`.
EXO_API int exo_gemm_bf16_swiglu_gated(const void* x, const void* W, void* out, int M, int N, int K, int parity, cudaStream_t st) {
  return gemm_swiglu_launch(x, W, out, M, N, K, parity, st);
}

static int gemm_swiglu_launch(const void* x, const void* W, void* out, int M, int N, int K, int gate_parity, cudaStream_t st) {
  if (M < 256 || (N & 1) || K % 8 != 0 || K < BK) return -2;
  int dev;
  cudaGetDevice(&dev);
  if (dev >= 16 || !g_err[dev]) return -4;
  const int bn = fit_rows((N / 2 + BM - 1) / BM, M);
  const CUtensorMap* tw = exo_tmap_2d_bf16(W, N, K, BM);
  const CUtensorMap* tx = exo_tmap_2d_bf16(x, M, K, bn);
  if (!tw || !tx) return -5;
  GemmParams p;
  memset(&p, 0, sizeof(p));
  p.M = M; p.N = N; p.K = K;
  p.kb_per_split = (K + BK - 1) / BK;
  p.bn_rows = bn;
  p.rows_fastest = rows_fastest_default();
  p.splits = 1;
  p.out = (__nv_bfloat16*)out;
  p.ldo = N / 2;
  p.err = g_err[dev];
  if (gate_parity >= 0) {
    int rc = gate_params(&p, gate_parity, M, bn);
    if (rc) return rc;
  }
  return launch_gemm_glu(tw, tx, p, st);
}

// Row-parallel projection whose [M, N] output goes into every rank's hand-over slot as flag-in-data words
// (see tp_handover.cuh); N even.
EXO_API int exo_gemm_bf16_tp(const void* x, const void* W, const void* bias, int M, int N, int K, int splits, int parity,
                             cudaStream_t st) {
  if (N & 1) return -2;
  TpHandover ho;
  int rc = exo_tp_handover_fill(&ho, 3, parity, (long)((M + 1) & ~1) * N);
  if (rc) return rc;
  return gemm_launch(x, W, bias, nullptr, nullptr, M, N, K, N, splits, &ho, st);
}

static int gemm_launch(const void* x, const void* W, const void* bias, const void* residual, void* out, int M, int N,
                       int K, int ldo, int splits, const TpHandover* ho, cudaStream_t st) {
  if (M <= 0 || N <= 0) return 0;
  if (K % 8 != 0 || K < BK) return -2;
  int dev;
  cudaGetDevice(&dev);
  if (dev >= 16 || !g_err[dev]) return -4;  // exo_gemm_init not called on this device
  int bn = M <= 16 ? 16 : M <= 32 ? 32 : M <= 64 ? 64 : M <= 128 ? 128 : 256;
  // prefill shapes: decide here whether the two-accumulator kernel runs, and with how many rows per CTA
  bool two = false;
  int fitted = 0;
  if (bn == 256 && splits <= 1 && !ho) {
    // Two accumulators per CTA halve the CTA count and make each ~1.74x as long (measured): take them when that
    // wins after both shapes got the row count that fits them best into whole waves over the 148 SMs.
    long c1 = 0, c2 = 0;
    const int r1 = fit_rows((N + BM - 1) / BM, M, &c1), r2 = fit_rows((N + 2 * BM - 1) / (2 * BM), M, &c2);
    static const bool single_tile = getenv("EXO_GEMM_SINGLE_TILE") != nullptr;   // A/B switch, read once
    two = N >= 2 * BM && !single_tile && 1.74 * (double)c2 < (double)c1;
    bn = fitted = two ? r2 : r1;
  }
  const CUtensorMap* tw = exo_tmap_2d_bf16(W, N, K, BM);
  const CUtensorMap* tx = exo_tmap_2d_bf16(x, M, K, bn);
  if (!tw || !tx) return -5;
  GemmParams p;
  memset(&p, 0, sizeof(p));
  p.M = M; p.N = N; p.K = K;
  p.bn_rows = fitted;
  p.rows_fastest = fitted > 0 && rows_fastest_default();
  int kb_total = (K + BK - 1) / BK;
  if (splits < 1) splits = 1;
  if (splits > kb_total) splits = kb_total;
  p.kb_per_split = (kb_total + splits - 1) / splits;
  splits = (kb_total + p.kb_per_split - 1) / p.kb_per_split;  // no empty split
  p.splits = splits;
  p.bias = (const __nv_bfloat16*)bias;
  p.residual = (const __nv_bfloat16*)residual;
  p.out = (__nv_bfloat16*)out;
  p.ldo = ldo;
  p.partial = g_partial[dev];
  p.counters = g_counters[dev];
  p.err = g_err[dev];
  if (ho) p.ho = *ho; else memset(&p.ho, 0, sizeof(p.ho));
  p.row_flags = nullptr; p.row_epoch = nullptr; p.rows_per_flag = 1; p.m_tile_shift = 0; p.gate_wait_ns = 0; p.gate_status = nullptr;
  if (g_gate_parity >= 0) {
    int rc = gate_params(&p, g_gate_parity, M, bn);
    if (rc) return rc;
  }
  if (splits > 1) {
    long tiles = (long)((N + BM - 1) / BM) * ((M + bn - 1) / bn);
    if ((size_t)splits * M * N > g_partial_floats[dev] || tiles > MAX_TILES) return -6;
  }
  if (two) return launch_gemm<256, 3, true>(tw, tx, p, st);   //  3 x 64 KB, two accumulators (512 TMEM columns)
  switch (bn) {
    case 16: return launch_gemm<16, 5>(tw, tx, p, st);   //  5 x 18 KB
    case 32: return launch_gemm<32, 5>(tw, tx, p, st);   //  5 x 20 KB
    case 64: return launch_gemm<64, 4>(tw, tx, p, st);   //  4 x 24 KB
    case 128: return launch_gemm<128, 3>(tw, tx, p, st); //  3 x 32 KB  (two CTAs per SM)
    default:
      return launch_gemm<256, 4>(tw, tx, p, st);  //  4 x 48 KB  (one CTA per SM)
  }
}
