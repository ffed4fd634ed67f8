// fp32 GEMM / SYRK on the 5th-generation tensor cores (tcgen05 + tensor memory)
// with an error-compensated 3xTF32 split.
//
//   a = a_hi + a_lo,  a*b ~= a_lo*b_hi + a_hi*b_lo + a_hi*b_hi     (a_lo*b_lo dropped)
//
// The tensor core reads an fp32 operand as TF32 by dropping the low 13 mantissa
// bits, so an operand whose rows are 16-byte aligned is used IN PLACE as its own
// hi part (a_hi = trunc_tf32(a), exact), and only a_lo = tf32(a - a_hi) is
// written to scratch by a small element-wise pre-pass.  A row-major B[K][N] is
// consumed as it lies (N-major operand, 128-byte swizzle with 32-byte atoms);
// the rank-k update's B = A^T is K-major like A.  Operands that break a TMA
// alignment rule get both planes written instead (B transposed on the way).
//
// The GEMM itself is one persistent, warp-specialised kernel (384 threads):
//   warp 0     TMA producer: four tile loads per K-block of 16 into a 4-stage
//              shared-memory ring (mbarrier transaction counts);
//   warp 1     one elected thread issues tcgen05.mma kind::tf32 (M=128, N=256,
//              K=8), six per K-block, accumulating in tensor memory;
//              tcgen05.commit releases ring stages and publishes accumulators;
//   warps 4-11 drain warps: tcgen05.ld the 128x256 fp32 accumulator (each thread
//              one row x 128 columns), add it into fp32 registers, and at the end
//              of a tile apply alpha/beta and store through a padded shared
//              32x32 transpose, so every access to C is a full 128-byte row
//              segment.
// setmaxnreg moves registers from warps 0-3 (40 each) to the drain warps (232).
// Tensor memory holds two accumulators, so the tensor cores work on chunk c+1
// (or the next tile) while chunk c is drained.  Problems with too few 128x256
// tiles to occupy the GPU run the same kernel with 128x64 tiles (N=64 MMAs,
// eight ring stages).
//
// Why chunks.  The tensor core adds each K=8 partial product into the fp32
// accumulator with truncation, which biases long all-positive sums (measured:
// -3.0e-4 relative at K=32768 in one accumulation).  Draining every
// `chunk_kblocks` K-blocks and adding the chunks in round-to-nearest fp32
// registers bounds that bias independently of K.  Each hand-off costs the tensor
// pipe about 0.3 us (the tensor-memory reads of the drain compete with the
// running MMAs), so the default of 8 K-blocks trades ~3e-6 of bias for ~5 % of
// time; 4 gives 2e-6 for ~13 %, 16 gives 5e-6 for ~2 %.
//
// Every wait is time-bounded: on expiry the kernel records a code in the
// host-visible status word, leaves its loops, frees its tensor memory and
// returns.
#include <vector>

#include "pgb200_internal.h"

namespace pgb200 {

namespace {

constexpr int BM = 128, BN = 256, BK = 16;
constexpr int STAGES = 4;
constexpr int A_BYTES = BM * BK * 4;                      // 8 KiB per plane tile
constexpr int B_BYTES = BN * BK * 4;                      // 16 KiB per plane tile
constexpr int STAGE_BYTES = 2 * A_BYTES + 2 * B_BYTES;    // 48 KiB
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024;
constexpr int EPI_WARPS = 8;
constexpr int FIRST_EPI_WARP = 4;                         // warps 0-3: producer, MMA, 2 spare
constexpr int THREADS = 32 * (FIRST_EPI_WARP + EPI_WARPS);
constexpr int TMEM_COLS = 512;
constexpr long long WAIT_CYCLES = 4000000000ll;           // ~2 s
constexpr long long STEP_WAIT_MIN = 200000ll;             // ~0.1 ms: least patience of the meeting between rounds
constexpr int DEFAULT_CHUNK_KBLOCKS = 8;                  // 128 K-elements

// ------------------------------------------------------------------ PTX helpers
__device__ __forceinline__ uint32_t smem_u32(const void *p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// Time-bounded wait: false when ~2 s of SM cycles passed without completion.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
  if (mbar_try(bar, parity)) return true;
  const long long t0 = clock64();
  for (;;) {
    for (int i = 0; i < 64; i++)
      if (mbar_try(bar, parity)) return true;
    if (clock64() - t0 > WAIT_CYCLES) return false;
  }
}
// Same, for waits entered by whole warps: sleeps between polls so that the
// spinning warps do not compete with the single MMA-issuing thread.
__device__ __forceinline__ bool mbar_wait_backoff(uint32_t bar, uint32_t parity) {
  // The accumulator hand-off is on the critical path of short chunks: poll
  // back to back for a while before starting to sleep between polls.
  for (int i = 0; i < 64; i++)
    if (mbar_try(bar, parity)) return true;
  const long long t0 = clock64();
  for (;;) {
    for (int i = 0; i < 16; i++) {
      __nanosleep(32);
      if (mbar_try(bar, parity)) return true;
    }
    if (clock64() - t0 > WAIT_CYCLES) return false;
  }
}
__device__ __forceinline__ void report_status(int32_t *status, int32_t code, int32_t detail) {
  volatile int32_t *s = status;
  s[1] = detail;
  s[0] = code;
  __threadfence_system();
}
// The TMA producers of a persistent grid meet between rounds of tiles (round r
// = tiles [r * CTAs, (r + 1) * CTAs) of the walk).  The tiles of a round share
// their A and B panels, and a panel (rows x K x hi+lo) is far larger than L2,
// so a CTA only finds a panel's lines in L2 while it walks K close behind the
// CTA that fetched them.  Left alone the CTAs drift apart over the rounds and
// most panel reads go to DRAM again (fp32 16384^3: 79-86 GB read against 44 GB
// with the meeting, which is what 74 tiles in step need); at the power cap the
// saved DRAM energy is SM clock (fp32 32768^3: 1155 -> 1455 MHz, 319 -> 268 ms).
// Each producer adds one to a zeroed counter when the loads of its tile are
// issued and waits for CTAs * r before round r.  The meeting is only a hint: a
// producer that has waited as long as a whole tile took goes on without the
// others (CTAs that started late, e.g. behind a short kernel of another
// stream, have caught up by the next round), and after the third such wait
// (the CTAs of the grid are not all running: another kernel holds some SMs)
// it stops meeting for good; the product is the same either way.
struct RoundMeeting {
  int32_t *ctr;
  bool waits;
  int32_t given_up;
  int32_t round;
  long long t_begin, tile_cycles;
  __device__ __forceinline__ void init(int32_t *counter) {
    ctr = counter;
    waits = counter != nullptr;
    given_up = 0;
    round = 0;
    t_begin = 0;
    tile_cycles = 0;
  }
  __device__ __forceinline__ void before_tile() {
    if (ctr == nullptr) return;
    t_begin = clock64();
    if (waits && round > 0) {
      const int32_t want = (int32_t)gridDim.x * round;
      const volatile int32_t *c = ctr;
      const long long limit = tile_cycles > STEP_WAIT_MIN ? tile_cycles : STEP_WAIT_MIN;
      while (*c < want) {
        if (clock64() - t_begin > limit) {
          if (++given_up >= 3) waits = false;
          break;
        }
        __nanosleep(100);
      }
    }
  }
  __device__ __forceinline__ void after_tile() {
    if (ctr == nullptr) return;
    atomicAdd(ctr, 1);
    tile_cycles = clock64() - t_begin;
    round++;
  }
};
// Pulls a tensor map into the descriptor cache ahead of its first use.
__device__ __forceinline__ void prefetch_tensor_map(const CUtensorMap *map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(map) : "memory");
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap *map, uint32_t bar,
                                            int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, "
      "{%3, %4}], [%2];" ::"r"(dst),
      "l"(map), "r"(bar), "r"(c0), "r"(c1)
      : "memory");
}
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap *map, uint32_t bar,
                                            int c0, int c1, int c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, "
      "{%3, %4, %5}], [%2];" ::"r"(dst),
      "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2)
      : "memory");
}
__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                   bar)
               : "memory");
}
__device__ __forceinline__ void tc_mma_tf32(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc,
                                            uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void tc_ld32(uint32_t taddr, uint32_t (&v)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]),
        "=r"(v[7]), "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]),
        "=r"(v[14]), "=r"(v[15]), "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]),
        "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]),
        "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tc_wait_ld() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// Shared-memory matrix descriptor of a K-major tile whose rows are one 64-byte
// swizzle span (16 fp32): 8-row groups are 512 bytes apart (stride byte offset),
// the leading byte offset is unused for swizzled K-major layouts, descriptor
// version 1 (sm_100), layout type 4 = 64-byte swizzle.
__device__ __forceinline__ uint64_t smem_desc_sw64(uint32_t saddr) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr & 0x3FFFFu) >> 4);        // start address, bits [0,14)
  d |= (uint64_t)1 << 16;                          // leading byte offset (ignored)
  d |= (uint64_t)((8 * BK * 4) >> 4) << 32;        // stride byte offset = 512 B
  d |= (uint64_t)1 << 46;                          // descriptor version
  d |= (uint64_t)4 << 61;                          // SWIZZLE_64B
  return d;
}

// Descriptor of an N-major ("MN-major") B tile, i.e. a row-major B[K][N] used as
// it lies: the tile is stored as 8 column blocks of 32 fp32 (one 128-byte
// span), each block [BK k-rows][128 bytes].  For 32-bit operands the tensor
// core takes N-major data only in the "128-byte swizzle with 32-byte atoms"
// layout (descriptor layout type 1; TMA mode SWIZZLE_128B_ATOM_32B), whose atom
// is 4 k-rows x 128 bytes.  Leading byte offset = distance between column
// blocks (BK*128), stride byte offset = distance between groups of 4 k-rows
// (512).  (Established with a one-tile probe: an identity-like A against
// B = k and B = n reproduces B exactly for this combination only.)
__device__ __forceinline__ uint64_t smem_desc_mn_sw128(uint32_t saddr) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr & 0x3FFFFu) >> 4);
  d |= (uint64_t)((BK * 128) >> 4) << 16;
  d |= (uint64_t)(512 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)1 << 61;
  return d;
}

// kind::tf32 instruction descriptor: fp32 accumulator, tf32 A and B, A K-major,
// B K-major (bit 16 clear) or N-major (bit 16 set), N=256, M=128.
constexpr uint32_t IDESC = (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(BN >> 3) << 17) |
                           ((uint32_t)(BM >> 4) << 24);
constexpr uint32_t IDESC_BMN = IDESC | (1u << 16);

// alpha/beta epilogue of one drain warp: `acc` holds, per thread, one row x COLS
// columns of the tile (row = r_base + lane, columns cb..cb+COLS-1).  Accessing C
// that way would touch 32 different rows per instruction, so the warp turns
// 32x32 blocks through a padded shared tile and reads/writes C as full 128-byte
// row segments (lane = column).  Interior blocks are software-pipelined: the 16
// loads of the next half-block are in flight while the current one is stored.
template <int COLS>
__device__ __forceinline__ void epilogue_store(const float (&acc)[COLS], float (*st)[33], int lane,
                                               int64_t r_base, int64_t cb, int64_t M, int64_t N,
                                               int64_t ldc, float *__restrict__ C, float alpha,
                                               float beta, bool lower, int64_t row0) {
  constexpr int NB = COLS / 32;
  const bool all_interior = (r_base + 31 < M) && (cb + COLS - 1 < N) &&
                            (!lower || cb + COLS - 1 <= r_base + row0);
  if (all_interior) {
    float *cptr = C + r_base * ldc + cb + lane;
    float cur[16], nxt[16];
    if (beta != 0.0f) {
#pragma unroll
      for (int q = 0; q < 16; q++) cur[q] = __ldcs(cptr + q * ldc);
    }
#pragma unroll
    for (int hb = 0; hb < 2 * NB; hb++) {
      const int blk = hb >> 1, h = hb & 1;
      if (h == 0) {
        __syncwarp();
#pragma unroll
        for (int i = 0; i < 32; i++) st[lane][i] = alpha * acc[blk * 32 + i];
        __syncwarp();
      }
      if (beta != 0.0f && hb + 1 < 2 * NB) {
        const int nblk = (hb + 1) >> 1, nh = (hb + 1) & 1;
#pragma unroll
        for (int q = 0; q < 16; q++) nxt[q] = __ldcs(cptr + nblk * 32 + (nh * 16 + q) * ldc);
      }
#pragma unroll
      for (int q = 0; q < 16; q++) {
        const float o = st[h * 16 + q][lane];
        cptr[blk * 32 + (h * 16 + q) * ldc] = (beta != 0.0f) ? fmaf(beta, cur[q], o) : o;
      }
#pragma unroll
      for (int q = 0; q < 16; q++) cur[q] = nxt[q];
    }
    return;
  }
  // Ragged edge or diagonal tile: block by block, element by element.
#pragma unroll
  for (int blk = 0; blk < NB; blk++) {
    if (cb + blk * 32 >= N) break;
    __syncwarp();
#pragma unroll
    for (int i = 0; i < 32; i++) st[lane][i] = alpha * acc[blk * 32 + i];
    __syncwarp();
    const int64_t c = cb + blk * 32 + lane;
    float *cptr = C + r_base * ldc + c;
#pragma unroll 4
    for (int rr = 0; rr < 32; rr++) {
      const int64_t r = r_base + rr;
      if (c < N && r < M && (!lower || c <= r + row0)) {
        float o = st[rr][lane];
        if (beta != 0.0f) o = fmaf(beta, cptr[rr * ldc], o);
        cptr[rr * ldc] = o;
      }
    }
  }
}

struct Tiles {
  int64_t tiles_m, tiles_n, total;
  int64_t row0;  // absolute row of local row 0 (lower only)
  int lower;
  int bn;        // tile width in columns (256, or 64 for problems with few tiles)
  int bm;        // tile height in rows (128; 256 for the two-CTA kernel's pair tiles)
  // A(i,k) is zero for k < i (two-CTA kernel only): the K loop of tile row tm
  // starts at its diagonal block, and odd rounds hand tiles out in reverse
  // order so every pair gets long and short tiles alike.
  int a_upper;
  // Split-K (one-CTA kernel, problems with few tiles): the K-blocks of a tile
  // are dealt to `splits` CTAs, `kper` each; CTA (tile, sp) writes its partial
  // product to partial[sp][M][ldp] and a second kernel adds them up in order.
  int splits;
  int64_t kper;
  float *partial;
  int64_t ldp;
  // Height of the bands the tile walk uses, in tile rows (0: the default of 16;
  // see TileCursor).  Measured at 16384^3 and 32768^3: bands of 8, 16 and 32 rows,
  // with and without an evict-last L2 policy on the loads of either operand,
  // all gave the same time within run-to-run noise and DRAM traffic within
  // +-10 %, so the walk is not what limits the large products.
  int band;
  // Products with more tiles than CTAs and a long K: the zeroed counter of the
  // meeting between rounds of tiles (see RoundMeeting); null: no meeting.
  int32_t *step_ctr;
  __device__ __forceinline__ int64_t first_kblock(int64_t tm) const {
    return a_upper ? (tm * bm) / BK : 0;
  }
  // May return an index >= total in the last round.
  __device__ __forceinline__ int64_t index(int64_t round, int64_t who, int64_t n) const {
    return round * n + ((a_upper && (round & 1)) ? n - 1 - who : who);
  }
};

// Columns tiles of tile-row tm that intersect j <= i (lower) or all of them.
__host__ __device__ __forceinline__ int64_t row_tiles(const Tiles &t, int64_t tm) {
  if (!t.lower) return t.tiles_n;
  const int64_t last_col = t.row0 + tm * t.bm + t.bm - 1;  // largest j of the tile row
  const int64_t c = last_col / t.bn + 1;
  return c < t.tiles_n ? c : t.tiles_n;
}

// Maps a linear tile index to (tile row, tile column).  Tiles are walked in
// bands of 16 tile-rows, column by column inside a band, so the ~148 tiles in
// flight form a 16 x 9 patch that shares 16 A panels and 9 B panels through L2
// instead of streaming every B panel in every wave.  For the triangular update
// only tiles that intersect j <= i exist; the band walk is the same, with each
// column holding only the rows that reach it.  Each role keeps its own cursor;
// tile indices only grow within a CTA, so the band position advances
// monotonically.
struct TileCursor {
  static constexpr int64_t G_DEFAULT = 16;
  int64_t band = 0, before = 0;  // tiles in bands < band (lower only)
  __host__ __device__ __forceinline__ void seek(const Tiles &t, int64_t idx, int64_t *otm,
                                                int64_t *otn) {
    const int64_t G = t.band > 0 ? t.band : G_DEFAULT;
    if (!t.lower) {
      const int64_t per_group = G * t.tiles_n;
      const int64_t grp = idx / per_group;
      const int64_t first = grp * G;
      const int64_t rows = (t.tiles_m - first < G) ? (t.tiles_m - first) : G;
      const int64_t in = idx - grp * per_group;
      *otm = first + in % rows;
      *otn = in / rows;
      return;
    }
    int64_t first, last;
    for (;;) {
      first = band * G;
      last = (first + G < t.tiles_m ? first + G : t.tiles_m) - 1;
      int64_t cnt = 0;
      for (int64_t r = first; r <= last; r++) cnt += row_tiles(t, r);
      if (idx < before + cnt) break;
      before += cnt;
      band++;
    }
    int64_t in = idx - before;
    for (int64_t tn = 0;; tn++) {
      // Smallest tile row whose last matrix row reaches column tile tn.
      int64_t need = tn * t.bn - t.row0 - (t.bm - 1);
      int64_t lo = need <= 0 ? 0 : (need + t.bm - 1) / t.bm;
      if (lo < first) lo = first;
      const int64_t c = last - lo + 1;
      if (c > 0) {
        if (in < c) {
          *otm = lo + in;
          *otn = tn;
          return;
        }
        in -= c;
      }
    }
  }
};

// Number of tiles the cursor enumerates (host side; the kernels get it in
// Tiles::total).
inline int64_t count_tiles(const Tiles &t) {
  int64_t total = 0;
  for (int64_t tm = 0; tm < t.tiles_m; tm++) total += row_tiles(t, tm);
  return total;
}

template <bool B_MN, int TBN, bool SPLITK>
__global__ void __launch_bounds__(THREADS, 1)
tf32x3_gemm_kernel(const __grid_constant__ CUtensorMap mapAhi,
                   const __grid_constant__ CUtensorMap mapAlo,
                   const __grid_constant__ CUtensorMap mapBhi,
                   const __grid_constant__ CUtensorMap mapBlo, int64_t M, int64_t N, int64_t K,
                   float alpha, float beta, float *__restrict__ C, int64_t ldc, Tiles tiles,
                   int chunk_kblocks, int bhi_blocked, int32_t *status) {
  // Tile-width dependent constants (these shadow the 256-wide defaults above).
  constexpr int BN = TBN;
  constexpr int B_BYTES = BN * BK * 4;
  constexpr int STAGE_BYTES = 2 * A_BYTES + 2 * B_BYTES;
  constexpr int STAGES = (192 * 1024) / STAGE_BYTES;  // 4 (BN=256) or 8 (BN=64)
  constexpr int COLS = BN / 2;                         // columns per drain thread
  constexpr uint32_t IDESC = (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(BN >> 3) << 17) |
                             ((uint32_t)(BM >> 4) << 24);
  constexpr uint32_t IDESC_BMN = IDESC | (1u << 16);
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t bars[2 * STAGES + 4];
  __shared__ uint32_t tmem_slot;
  __shared__ float epi_stage[EPI_WARPS][32][33];
  const uint32_t ring = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t full0 = smem_u32(&bars[0]), empty0 = smem_u32(&bars[STAGES]);
  const uint32_t accf0 = smem_u32(&bars[2 * STAGES]), acce0 = smem_u32(&bars[2 * STAGES + 2]);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 64) {  // an otherwise idle warp
    prefetch_tensor_map(&mapAhi);
    prefetch_tensor_map(&mapAlo);
    prefetch_tensor_map(&mapBhi);
    prefetch_tensor_map(&mapBlo);
  }
  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; s++) {
      mbar_init(full0 + 8 * s, 1);
      mbar_init(empty0 + 8 * s, 1);
    }
    for (int b = 0; b < 2; b++) {
      mbar_init(accf0 + 8 * b, 1);
      mbar_init(acce0 + 8 * b, EPI_WARPS);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     smem_u32(&tmem_slot)),
                 "r"(TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_slot;

  // Register re-partition between the warpgroups: the producer/MMA group keeps
  // 40 registers per thread, the two drain groups (128 fp32 accumulators per
  // thread plus tensor-memory load buffers) grow to 232.
  const int64_t nkb = (K + BK - 1) / BK;
  const int64_t nchunks = (nkb + chunk_kblocks - 1) / chunk_kblocks;
  const int64_t work = SPLITK ? tiles.total * tiles.splits : tiles.total;  // (tile, K range) items

  if (warp < FIRST_EPI_WARP) {
  // Register re-partition between the warpgroups: the producer/MMA group gives
  // registers back, the two drain groups (128 fp32 accumulators per thread plus
  // tensor-memory load buffers) grow.
  asm volatile("setmaxnreg.dec.sync.aligned.u32 40;");
  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      TileCursor cur;
      uint32_t stage = 0, phase = 0;
      bool ok = true;
      RoundMeeting meeting;
      meeting.init(SPLITK ? nullptr : tiles.step_ctr);
      for (int64_t w = blockIdx.x; w < work && ok; w += gridDim.x) {
        const int64_t t = SPLITK ? w / tiles.splits : w;
        const int64_t kb_lo = SPLITK ? (w % tiles.splits) * tiles.kper : 0;
        const int64_t kb_hi = SPLITK ? (kb_lo + tiles.kper < nkb ? kb_lo + tiles.kper : nkb) : nkb;
        int64_t tm, tn;
        cur.seek(tiles, t, &tm, &tn);
        meeting.before_tile();
        for (int64_t kb = kb_lo; kb < kb_hi; kb++) {
          if (!mbar_wait(empty0 + 8 * stage, phase ^ 1)) {
            report_status(status, 11, (int32_t)blockIdx.x);
            ok = false;
            break;
          }
          const uint32_t dst = ring + stage * STAGE_BYTES;
          const uint32_t bar = full0 + 8 * stage;
          mbar_expect_tx(bar, STAGE_BYTES);
          const int k0 = (int)(kb * BK);
          tma_load_2d(dst, &mapAhi, bar, k0, (int)(tm * BM));
          tma_load_2d(dst + A_BYTES, &mapAlo, bar, k0, (int)(tm * BM));
          if (B_MN) {
            // Row-major B as it lies: eight [BK x 32] column blocks per plane,
            // fetched by one 3-D copy (view (32, K, N/32)) when N allows it,
            // else by eight 2-D copies (zero-filled past column N).
            tma_load_3d(dst + 2 * A_BYTES + B_BYTES, &mapBlo, bar, 0, k0, (int)(tn * (BN / 32)));
            if (bhi_blocked) {
              tma_load_3d(dst + 2 * A_BYTES, &mapBhi, bar, 0, k0, (int)(tn * (BN / 32)));
            } else {
#pragma unroll
              for (int j = 0; j < BN / 32; j++)
                tma_load_2d(dst + 2 * A_BYTES + j * (BK * 128), &mapBhi, bar,
                            (int)(tn * BN) + 32 * j, k0);
            }
          } else {
            tma_load_2d(dst + 2 * A_BYTES, &mapBhi, bar, k0, (int)(tn * BN));
            tma_load_2d(dst + 2 * A_BYTES + B_BYTES, &mapBlo, bar, k0, (int)(tn * BN));
          }
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
        meeting.after_tile();
      }
    }
  } else if (warp == 1) {
    // -------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      uint32_t stage = 0, phase = 0;
      int64_t cc = 0;  // chunks issued by this CTA so far
      bool ok = true;
      for (int64_t w = blockIdx.x; w < work && ok; w += gridDim.x) {
        const int64_t kb_lo = SPLITK ? (w % tiles.splits) * tiles.kper : 0;
        const int64_t kb_hi = SPLITK ? (kb_lo + tiles.kper < nkb ? kb_lo + tiles.kper : nkb) : nkb;
        const int64_t nch = SPLITK ? (kb_hi - kb_lo + chunk_kblocks - 1) / chunk_kblocks : nchunks;
        for (int64_t ch = 0; ch < nch && ok; ch++, cc++) {
          const uint32_t buf = (uint32_t)(cc & 1);
          const uint32_t use = (uint32_t)((cc >> 1) & 1);
          if (!mbar_wait(acce0 + 8 * buf, use ^ 1)) {
            report_status(status, 12, (int32_t)blockIdx.x);
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t tmem_d = tmem_base + buf * BN;
          const int64_t kb_first = kb_lo + ch * chunk_kblocks;
          const int64_t kb_end = kb_first + chunk_kblocks < kb_hi ? kb_first + chunk_kblocks : kb_hi;
          for (int64_t kb = kb_first; kb < kb_end; kb++) {
            if (!mbar_wait(full0 + 8 * stage, phase)) {
              report_status(status, 13, (int32_t)blockIdx.x);
              ok = false;
              break;
            }
            tc_fence_after();
            const uint32_t sa = ring + stage * STAGE_BYTES;
            const uint64_t ahi = smem_desc_sw64(sa), alo = smem_desc_sw64(sa + A_BYTES);
            const uint64_t bhi = B_MN ? smem_desc_mn_sw128(sa + 2 * A_BYTES)
                                      : smem_desc_sw64(sa + 2 * A_BYTES);
            const uint64_t blo = B_MN ? smem_desc_mn_sw128(sa + 2 * A_BYTES + B_BYTES)
                                      : smem_desc_sw64(sa + 2 * A_BYTES + B_BYTES);
            constexpr uint32_t idesc = B_MN ? IDESC_BMN : IDESC;
            const bool first = (kb == kb_first);
#pragma unroll
            for (int ks = 0; ks < BK / 8; ks++) {
              // K=8 step: +32 bytes inside a K-major swizzled row; one group of
              // 8 k-rows (+1024 bytes) in an N-major tile (both encoded >> 4).
              const uint64_t ko = (uint64_t)(ks * 2);
              const uint64_t kob = B_MN ? (uint64_t)(ks * 64) : ko;
              tc_mma_tf32(tmem_d, alo + ko, bhi + kob, idesc, (first && ks == 0) ? 0u : 1u);
              tc_mma_tf32(tmem_d, ahi + ko, blo + kob, idesc, 1u);
              tc_mma_tf32(tmem_d, ahi + ko, bhi + kob, idesc, 1u);
            }
            tc_commit(empty0 + 8 * stage);  // stage reusable once these MMAs retire
            if (++stage == STAGES) {
              stage = 0;
              phase ^= 1;
            }
          }
          if (ok) tc_commit(accf0 + 8 * buf);  // accumulator complete
        }
      }
    }
  }
  } else {
    // ------------------------------------------------------------- drain warps
    asm volatile("setmaxnreg.inc.sync.aligned.u32 232;");
    const int ew = warp - FIRST_EPI_WARP;
    const int quarter = warp & 3;      // tensor-memory lane quarter this warp may read
    const int half = ew >> 2;          // which half of the tile's columns
    TileCursor cur;
    int64_t cc = 0;
    bool ok = true;
    for (int64_t w = blockIdx.x; w < work && ok; w += gridDim.x) {
      const int64_t t = SPLITK ? w / tiles.splits : w;
      const int64_t sp = SPLITK ? w % tiles.splits : 0;
      const int64_t kb_lo = SPLITK ? sp * tiles.kper : 0;
      const int64_t kb_hi = SPLITK ? (kb_lo + tiles.kper < nkb ? kb_lo + tiles.kper : nkb) : nkb;
      const int64_t nch = SPLITK ? (kb_hi - kb_lo + chunk_kblocks - 1) / chunk_kblocks : nchunks;
      int64_t tm, tn;
      cur.seek(tiles, t, &tm, &tn);
      float acc[COLS];
#pragma unroll
      for (int i = 0; i < COLS; i++) acc[i] = 0.0f;
      if (!SPLITK && beta != 0.0f) {
        // Pull this thread's part of the C tile towards L2 while the tensor
        // cores work, so the epilogue's loads do not wait on HBM.
        const int64_t pr = tm * BM + quarter * 32 + lane, pc = tn * BN + half * COLS;
        if (pr < M) {
#pragma unroll
          for (int q = 0; q < COLS / 32; q++)
            if (pc + q * 32 < N)
              asm volatile("prefetch.global.L2 [%0];" ::"l"(C + pr * ldc + pc + q * 32));
        }
      }
      for (int64_t ch = 0; ch < nch && ok; ch++, cc++) {
        const uint32_t buf = (uint32_t)(cc & 1);
        const uint32_t use = (uint32_t)((cc >> 1) & 1);
        if (!mbar_wait_backoff(accf0 + 8 * buf, use)) {
          if (lane == 0) report_status(status, 14, (int32_t)blockIdx.x);
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t taddr =
            tmem_base + ((uint32_t)(quarter * 32) << 16) + buf * BN + (uint32_t)(half * COLS);
#pragma unroll
        for (int j = 0; j < COLS / 32; j += 2) {
          uint32_t v0[32], v1[32];
          tc_ld32(taddr + j * 32, v0);
          if (j + 1 < COLS / 32) tc_ld32(taddr + j * 32 + 32, v1);
          tc_wait_ld();
#pragma unroll
          for (int i = 0; i < 32; i++) acc[j * 32 + i] += __uint_as_float(v0[i]);
          if (j + 1 < COLS / 32) {
#pragma unroll
            for (int i = 0; i < 32; i++) acc[j * 32 + 32 + i] += __uint_as_float(v1[i]);
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(acce0 + 8 * buf);
      }
      if (!ok) break;

      if (SPLITK)  // raw partial product of this K range; scaled and added up afterwards
        epilogue_store<COLS>(acc, epi_stage[ew], lane, tm * BM + quarter * 32,
                             tn * BN + half * COLS, M, N, tiles.ldp,
                             tiles.partial + sp * M * tiles.ldp, 1.0f, 0.0f, false, 0);
      else
        epilogue_store<COLS>(acc, epi_stage[ew], lane, tm * BM + quarter * 32,
                             tn * BN + half * COLS, M, N, ldc, C, alpha, beta, tiles.lower != 0,
                             tiles.row0);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                 "r"(TMEM_COLS)
                 : "memory");
  }
}

// C = beta*C + alpha*(P[0] + P[1] + ...), the partial products of a split-K
// launch added in a fixed order (four columns per thread).
constexpr int MAX_SPLITS = 8;
__global__ void splitk_reduce_kernel(const float *__restrict__ P, int64_t ldp, int splits, int64_t M,
                                     int64_t N, float alpha, float beta, float *__restrict__ C,
                                     int64_t ldc, int lower, int64_t row0) {
  const int64_t quads = ldp / 4;
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= M * quads) return;
  const int64_t r = i / quads, c = (i - r * quads) * 4;
  // lower: row r is absolute row r + row0 and owns columns up to it.
  const int64_t lim = lower ? (r + row0 < N - 1 ? r + row0 : N - 1) : N - 1;
  if (c > lim) return;
  // All loads first (independent, up to MAX_SPLITS of them in flight), then the
  // sum in split order.
  float4 v[MAX_SPLITS];
  const float *src = P + r * ldp + c;
#pragma unroll
  for (int sp = 0; sp < MAX_SPLITS; sp++)
    if (sp < splits) v[sp] = __ldcs(reinterpret_cast<const float4 *>(src + (int64_t)sp * M * ldp));
  float old[4] = {0.0f, 0.0f, 0.0f, 0.0f};
  float *dst = C + r * ldc + c;
  if (beta != 0.0f) {
#pragma unroll
    for (int j = 0; j < 4; j++)
      if (c + j <= lim) old[j] = dst[j];
  }
  float4 sum = v[0];
#pragma unroll
  for (int sp = 1; sp < MAX_SPLITS; sp++)
    if (sp < splits) {
      sum.x += v[sp].x;
      sum.y += v[sp].y;
      sum.z += v[sp].z;
      sum.w += v[sp].w;
    }
  const float part[4] = {sum.x, sum.y, sum.z, sum.w};
#pragma unroll
  for (int j = 0; j < 4; j++) {
    if (c + j > lim) break;
    const float o = alpha * part[j];
    dst[j] = (beta != 0.0f) ? fmaf(beta, old[j], o) : o;
  }
}

// ------------------------------------------------------------------ split kernels
__device__ __forceinline__ void split_tf32(float a, float *hi, float *lo) {
  uint32_t h, l;
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(h) : "f"(a));
  const float hf = __uint_as_float(h);
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(l) : "f"(a - hf));
  *hi = hf;
  *lo = __uint_as_float(l);
}

// src[rows][K] (ld) -> hi/lo[rows][Kp]; columns K..Kp-1 are zero-filled.
__global__ void split_rows_kernel(const float *__restrict__ src, int64_t ld, int64_t rows,
                                  int64_t K, int64_t Kp, float *__restrict__ hi,
                                  float *__restrict__ lo) {
  const int64_t total = rows * Kp;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total;
       i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = i / Kp, k = i - r * Kp;
    float h = 0.0f, l = 0.0f;
    if (k < K) split_tf32(src[r * ld + k], &h, &l);
    hi[i] = h;
    lo[i] = l;
  }
}

// The tensor core reads an fp32 operand as TF32 by dropping the low 13 mantissa
// bits, so an aligned operand can serve as its own "hi" plane: only
// lo = tf32(a - trunc_tf32(a)) has to be written.  src[rows][cols] (ld) ->
// lo[rows][colsP]; columns cols..colsP-1 are zero-filled.  Needs ld % 4 == 0
// and a 16-byte aligned src (the condition for using src as the hi plane).
__device__ __forceinline__ void split_lo_range(const float *__restrict__ src, int64_t ld,
                                               int64_t rows, int64_t cols, int64_t colsP,
                                               float *__restrict__ lo, int64_t first,
                                               int64_t stride) {
  const int64_t q = colsP / 4;  // float4 groups per row
  const int64_t total = rows * q;
  for (int64_t i = first; i < total; i += stride) {
    const int64_t r = i / q, c = (i - r * q) * 4;
    float v[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    if (c + 3 < cols) {
      const float4 x = *reinterpret_cast<const float4 *>(src + r * ld + c);
      v[0] = x.x; v[1] = x.y; v[2] = x.z; v[3] = x.w;
    } else {
      for (int e = 0; e < 4; e++)
        if (c + e < cols) v[e] = src[r * ld + c + e];
    }
    float o[4];
#pragma unroll
    for (int e = 0; e < 4; e++) {
      const float hi = __uint_as_float(__float_as_uint(v[e]) & 0xFFFFE000u);
      uint32_t l;
      asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(l) : "f"(v[e] - hi));
      o[e] = __uint_as_float(l);
    }
    *reinterpret_cast<float4 *>(lo + r * colsP + c) = make_float4(o[0], o[1], o[2], o[3]);
  }
}

__global__ void split_lo_kernel(const float *__restrict__ src, int64_t ld, int64_t rows,
                                int64_t cols, int64_t colsP, float *__restrict__ lo) {
  split_lo_range(src, ld, rows, cols, colsP, lo, blockIdx.x * (int64_t)blockDim.x + threadIdx.x,
                 (int64_t)gridDim.x * blockDim.x);
}

// Both operands in one launch: blocks [0,blocks0) take the first, the rest the second.
__global__ void split_lo_pair_kernel(const float *__restrict__ src0, int64_t ld0, int64_t rows0,
                                     int64_t cols0, int64_t colsP0, float *__restrict__ lo0,
                                     int blocks0, const float *__restrict__ src1, int64_t ld1,
                                     int64_t rows1, int64_t cols1, int64_t colsP1,
                                     float *__restrict__ lo1) {
  if ((int)blockIdx.x < blocks0)
    split_lo_range(src0, ld0, rows0, cols0, colsP0, lo0,
                   blockIdx.x * (int64_t)blockDim.x + threadIdx.x, (int64_t)blocks0 * blockDim.x);
  else
    split_lo_range(src1, ld1, rows1, cols1, colsP1, lo1,
                   (blockIdx.x - blocks0) * (int64_t)blockDim.x + threadIdx.x,
                   (int64_t)(gridDim.x - blocks0) * blockDim.x);
}

// src[K][N] (ld) -> hi/lo[N][Kp] (transposed through a 32x33 shared tile).
__global__ void split_transpose_kernel(const float *__restrict__ src, int64_t ld, int64_t K,
                                       int64_t N, int64_t Kp, float *__restrict__ hi,
                                       float *__restrict__ lo, int64_t tiles_k) {
  __shared__ float tile[32][33];
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;  // 32 x 8
  const int64_t tk = blockIdx.x % tiles_k, tn = blockIdx.x / tiles_k;
  const int64_t k0 = tk * 32, n0 = tn * 32;
#pragma unroll
  for (int i = 0; i < 4; i++) {
    const int64_t k = k0 + ty + 8 * i, n = n0 + tx;
    tile[ty + 8 * i][tx] = (k < K && n < N) ? src[k * ld + n] : 0.0f;
  }
  __syncthreads();
#pragma unroll
  for (int i = 0; i < 4; i++) {
    const int64_t n = n0 + ty + 8 * i, k = k0 + tx;
    if (n < N && k < Kp) {
      float h, l;
      split_tf32(tile[tx][ty + 8 * i], &h, &l);
      hi[n * Kp + k] = h;
      lo[n * Kp + k] = l;
    }
  }
}

// K-major operand [rows][K] with row pitch `ld`: box = BK x box_rows, 64-byte swizzle.
int32_t make_plane_map(CUtensorMap *map, const float *base, int64_t rows, int64_t K, int64_t ld,
                       int box_rows) {
  const uint64_t dims[2] = {(uint64_t)K, (uint64_t)rows};
  const uint64_t str[1] = {(uint64_t)ld * 4};
  const uint32_t box[2] = {BK, (uint32_t)box_rows};
  return encode_tensor_map(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, base, dims, str, box,
                           CU_TENSOR_MAP_SWIZZLE_64B);
}

// N-major operand B[K][N] with row pitch `ld`: box = 32 columns x BK rows,
// 128-byte swizzle with 32-byte atoms.
int32_t make_nmajor_map(CUtensorMap *map, const float *base, int64_t K, int64_t N, int64_t ld) {
  const uint64_t dims[2] = {(uint64_t)N, (uint64_t)K};
  const uint64_t str[1] = {(uint64_t)ld * 4};
  const uint32_t box[2] = {32, BK};
  return encode_tensor_map(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, base, dims, str, box,
                           CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B);
}

// The same operand seen as (32, K, N/32) so that one copy fetches all eight
// column blocks of a tile; needs N % 32 == 0 (every block inside the row).
int32_t make_nmajor_map_blocked(CUtensorMap *map, const float *base, int64_t K, int64_t N,
                                int64_t ld, int bn) {
  const uint64_t dims[3] = {32, (uint64_t)K, (uint64_t)(N / 32)};
  const uint64_t str[2] = {(uint64_t)ld * 4, 128};
  const uint32_t box[3] = {32, BK, (uint32_t)(bn / 32)};
  return encode_tensor_map(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, base, dims, str, box,
                           CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B);
}


// Tensor-pipe peak probe: every CTA issues `iters` back-to-back kind::tf32 MMAs
// (M=128, N=256, K=8) on whatever its shared memory holds and waits for them.
__global__ void __launch_bounds__(128, 1) tf32_probe_kernel(int iters, int32_t *status) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t bar;
  __shared__ uint32_t tmem_slot;
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    mbar_init(smem_u32(&bar), 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     smem_u32(&tmem_slot)),
                 "r"(TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  // Finite operand data so that the accumulators stay finite.
  for (int i = threadIdx.x; i < (A_BYTES + B_BYTES) / 4; i += blockDim.x)
    reinterpret_cast<float *>(smem_raw + (base - smem_u32(smem_raw)))[i] = 1.0f / (float)(1 + (i & 7));
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_slot;
  if (warp == 0 && lane == 0) {
    const uint64_t a = smem_desc_sw64(base), b = smem_desc_sw64(base + A_BYTES);
    for (int i = 0; i < iters; i++)
      tc_mma_tf32(tmem_base + (uint32_t)((i & 1) * BN), a + (uint64_t)((i & 1) * 2),
                  b + (uint64_t)((i & 1) * 2), IDESC, i < 2 ? 0u : 1u);
    tc_commit(smem_u32(&bar));
    if (!mbar_wait(smem_u32(&bar), 0)) report_status(status, 21, (int32_t)blockIdx.x);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                 "r"(TMEM_COLS)
                 : "memory");
  }
}

}  // namespace

// ===========================================================================
// Two-CTA variant (cta_group::2) of the same pipeline: every product with at
// least 512 rows and enough 128x256 tiles to fill the GPU.
//
// A cluster of two CTAs on an SM pair shares one 256x256 output tile: CTA r
// holds rows [128r, 128r+128) of the tile's A panel and columns
// [128r, 128r+128) of its B panel, and the accumulator rows of its own half in
// its own tensor memory.  One thread of the leader CTA (rank 0) issues
// tcgen05.mma.cta_group::2 (M=256, N=256, K=8); the tensor cores of both SMs
// read A from their own shared memory and B from both.  Per CTA a K-block
// stage is therefore 32 KiB instead of 48 KiB (each B column is fetched by one
// of the two SMs only), which buys two more ring stages and a third less
// L2 -> SM traffic.
//
// Hand-offs: both CTAs' TMA loads signal the leader's "full" barrier
// (cp.async.bulk.tensor...cta_group::2 with the barrier address's CTA bit
// cleared; no multicast load is used); the leader's tcgen05.commit arrives on
// the "empty" / "accumulator ready" barriers of both CTAs (commit multicast);
// the peer's drain warps arrive on the leader's "accumulator drained" barrier
// through its cluster address.  All waits are time-bounded and every thread of
// both CTAs reaches the two cluster barriers (start, end) unconditionally.
// ===========================================================================
namespace {

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Address of the same shared-memory offset in CTA `rank` of the cluster.
__device__ __forceinline__ uint32_t map_to_cta(uint32_t addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr)
               : "memory");
}
__device__ __forceinline__ void tma2_load_2d(uint32_t dst, const CUtensorMap *map,
                                             uint32_t leader_bar, int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%3, %4}], [%2];" ::"r"(dst),
      "l"(map), "r"(leader_bar), "r"(c0), "r"(c1)
      : "memory");
}
__device__ __forceinline__ void tma2_load_3d(uint32_t dst, const CUtensorMap *map,
                                             uint32_t leader_bar, int c0, int c1, int c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%3, %4, %5}], [%2];" ::"r"(dst),
      "l"(map), "r"(leader_bar), "r"(c0), "r"(c1), "r"(c2)
      : "memory");
}
__device__ __forceinline__ void tc2_mma_tf32(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc,
                                             uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::tf32 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Arrives on the barrier at this offset in both CTAs of the pair once all
// earlier MMAs of this thread have retired.
__device__ __forceinline__ void tc2_commit_both(uint32_t bar) {
  asm volatile(
      "{\n\t.reg .b16 m;\n\t"
      "mov.b16 m, 3;\n\t"
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 "
      "[%0], m;\n\t}" ::"r"(bar)
      : "memory");
}

// Optional host-built tile schedule of the triangular variant (an empty
// parameter for the dense one).
template <bool ON>
struct SchedParam {};
template <>
struct SchedParam<true> {
  int use;  // 0: round-robin with reversed odd rounds
  TileSchedule s;
};

// Turn `it` of CTA pair `pair`: is there one, and which tile (-1: none this turn).
template <bool A_UPPER>
__device__ __forceinline__ bool p2_more(const SchedParam<A_UPPER> &sp, int64_t it, int64_t pair,
                                        int64_t npairs, int64_t total) {
  if constexpr (A_UPPER) {
    if (sp.use) return (int64_t)sp.s.off[pair] + it < (int64_t)sp.s.off[pair + 1];
    return it * npairs < total;
  } else {
    return it < total;
  }
}
template <bool A_UPPER>
__device__ __forceinline__ int64_t p2_tile(const SchedParam<A_UPPER> &sp, const Tiles &tiles,
                                           int64_t it, int64_t pair, int64_t npairs,
                                           int64_t total) {
  if constexpr (A_UPPER) {
    if (sp.use) return sp.s.idx[(int64_t)sp.s.off[pair] + it];
    const int64_t x = tiles.index(it, pair, npairs);
    return x < total ? x : -1;
  } else {
    return it;
  }
}

template <bool B_MN, bool A_UPPER, int PN>
__global__ void __launch_bounds__(THREADS, 1)
tf32x3_gemm_2cta_kernel(const __grid_constant__ CUtensorMap mapAhi,
                        const __grid_constant__ CUtensorMap mapAlo,
                        const __grid_constant__ CUtensorMap mapBhi,
                        const __grid_constant__ CUtensorMap mapBlo, int64_t M, int64_t N,
                        int64_t K, float alpha, float beta, float *__restrict__ C, int64_t ldc,
                        Tiles tiles, int chunk_kblocks,
                        const __grid_constant__ SchedParam<A_UPPER> sp, int32_t *status) {
  // Pair tile of 256 rows x PN columns (256, or 128 for problems with few
  // tiles); each CTA holds PN/2 of the B columns.
  static_assert(PN == 256 || PN == 128, "pair tile width");
  constexpr int P2_BNH = PN / 2;
  constexpr int P2_B_BYTES = P2_BNH * BK * 4;
  constexpr int P2_STAGE_BYTES = 2 * A_BYTES + 2 * P2_B_BYTES;  // 32 or 24 KiB per CTA
  constexpr int P2_STAGES = (192 * 1024) / P2_STAGE_BYTES;      // 6 or 8
  constexpr uint32_t P2_IDESC = (1u << 4) | (2u << 7) | (2u << 10) |
                                ((uint32_t)(PN >> 3) << 17) | ((uint32_t)(256 >> 4) << 24);
  constexpr int COLS = PN / 2;  // columns per drain thread
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t bars[2 * P2_STAGES + 4];
  __shared__ uint32_t tmem_slot;
  __shared__ float epi_stage[EPI_WARPS][32][33];
  const uint32_t ring = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t full0 = smem_u32(&bars[0]), empty0 = smem_u32(&bars[P2_STAGES]);
  const uint32_t accf0 = smem_u32(&bars[2 * P2_STAGES]);
  const uint32_t acce0 = smem_u32(&bars[2 * P2_STAGES + 2]);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const int64_t pair = blockIdx.x >> 1, npairs = gridDim.x >> 1;
  const int64_t total = tiles.total;  // pair tiles of 256 x PN (tiles.bm == 256, tiles.bn == PN)

  if (threadIdx.x == 64) {  // an otherwise idle warp
    prefetch_tensor_map(&mapAhi);
    prefetch_tensor_map(&mapAlo);
    prefetch_tensor_map(&mapBhi);
    prefetch_tensor_map(&mapBlo);
  }
  if (threadIdx.x == 0) {
    for (int s = 0; s < P2_STAGES; s++) {
      mbar_init(full0 + 8 * s, 1);   // the leader's arrive.expect_tx (bytes of both CTAs)
      mbar_init(empty0 + 8 * s, 1);  // one commit arrival per CTA
    }
    for (int b = 0; b < 2; b++) {
      mbar_init(accf0 + 8 * b, 1);
      mbar_init(acce0 + 8 * b, 2 * EPI_WARPS);  // drain warps of both CTAs (leader's copy is used)
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     smem_u32(&tmem_slot)),
                 "r"(TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  cluster_sync_all();
  tc_fence_after();
  const uint32_t tmem_base = tmem_slot;

  const int64_t nkb = (K + BK - 1) / BK;
  if (warp < FIRST_EPI_WARP) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 40;");
    if (warp == 0) {
      // ------------------------------------------------ TMA producer (both CTAs)
      if (lane == 0) {
        uint32_t stage = 0, phase = 0;
        bool ok = true;
        const uint32_t leader_full0 = map_to_cta(full0, 0);
        TileCursor cur;
        RoundMeeting meeting;
        meeting.init(A_UPPER ? nullptr : tiles.step_ctr);
        for (int64_t it = A_UPPER ? 0 : pair; p2_more<A_UPPER>(sp, it, pair, npairs, total) && ok;
             it += A_UPPER ? 1 : npairs) {
          const int64_t t = p2_tile<A_UPPER>(sp, tiles, it, pair, npairs, total);
          if (A_UPPER && t < 0) continue;
          meeting.before_tile();
          int64_t tm2, tn;
          cur.seek(tiles, t, &tm2, &tn);
          const int row_a = (int)(tm2 * 256 + rank * 128);
          const int col_b = (int)(tn * PN + rank * P2_BNH);
          for (int64_t kb = A_UPPER ? tiles.first_kblock(tm2) : 0; kb < nkb; kb++) {
            if (!mbar_wait(empty0 + 8 * stage, phase ^ 1)) {
              report_status(status, 31, (int32_t)blockIdx.x);
              ok = false;
              break;
            }
            const uint32_t dst = ring + stage * P2_STAGE_BYTES;
            if (rank == 0) mbar_expect_tx(full0 + 8 * stage, 2 * P2_STAGE_BYTES);
            // The same barrier in the leader CTA, as a cluster address.
            const uint32_t lbar = leader_full0 + 8 * stage;
            const int k0 = (int)(kb * BK);
            tma2_load_2d(dst, &mapAhi, lbar, k0, row_a);
            tma2_load_2d(dst + A_BYTES, &mapAlo, lbar, k0, row_a);
            if (B_MN) {
              tma2_load_3d(dst + 2 * A_BYTES, &mapBhi, lbar, 0, k0, col_b / 32);
              tma2_load_3d(dst + 2 * A_BYTES + P2_B_BYTES, &mapBlo, lbar, 0, k0, col_b / 32);
            } else {
              tma2_load_2d(dst + 2 * A_BYTES, &mapBhi, lbar, k0, col_b);
              tma2_load_2d(dst + 2 * A_BYTES + P2_B_BYTES, &mapBlo, lbar, k0, col_b);
            }
            if (++stage == P2_STAGES) {
              stage = 0;
              phase ^= 1;
            }
          }
          meeting.after_tile();
        }
      }
    } else if (warp == 1 && rank == 0) {
      // ------------------------------------------------ MMA issuer (leader only)
      if (lane == 0) {
        uint32_t stage = 0, phase = 0;
        int64_t cc = 0;
        bool ok = true;
        TileCursor cur;
        for (int64_t it = A_UPPER ? 0 : pair; p2_more<A_UPPER>(sp, it, pair, npairs, total) && ok;
             it += A_UPPER ? 1 : npairs) {
          const int64_t t = p2_tile<A_UPPER>(sp, tiles, it, pair, npairs, total);
          if (A_UPPER && t < 0) continue;
          int64_t kb0 = 0;
          if (A_UPPER) {
            int64_t tm2, tn;
            cur.seek(tiles, t, &tm2, &tn);
            kb0 = tiles.first_kblock(tm2);
          }
          const int64_t nchunks = (nkb - kb0 + chunk_kblocks - 1) / chunk_kblocks;
          for (int64_t ch = 0; ch < nchunks && ok; ch++, cc++) {
            const uint32_t buf = (uint32_t)(cc & 1);
            const uint32_t use = (uint32_t)((cc >> 1) & 1);
            if (!mbar_wait(acce0 + 8 * buf, use ^ 1)) {
              report_status(status, 32, (int32_t)blockIdx.x);
              ok = false;
              break;
            }
            tc_fence_after();
            const uint32_t tmem_d = tmem_base + buf * PN;
            const int64_t kb_first = kb0 + ch * chunk_kblocks;
            const int64_t kb_end = kb_first + chunk_kblocks < nkb ? kb_first + chunk_kblocks : nkb;
            for (int64_t kb = kb_first; kb < kb_end; kb++) {
              if (!mbar_wait(full0 + 8 * stage, phase)) {
                report_status(status, 33, (int32_t)blockIdx.x);
                ok = false;
                break;
              }
              tc_fence_after();
              const uint32_t sa = ring + stage * P2_STAGE_BYTES;
              const uint64_t ahi = smem_desc_sw64(sa), alo = smem_desc_sw64(sa + A_BYTES);
              const uint64_t bhi = B_MN ? smem_desc_mn_sw128(sa + 2 * A_BYTES)
                                        : smem_desc_sw64(sa + 2 * A_BYTES);
              const uint64_t blo = B_MN ? smem_desc_mn_sw128(sa + 2 * A_BYTES + P2_B_BYTES)
                                        : smem_desc_sw64(sa + 2 * A_BYTES + P2_B_BYTES);
              constexpr uint32_t idesc = B_MN ? (P2_IDESC | (1u << 16)) : P2_IDESC;
              const bool first = (kb == kb_first);
#pragma unroll
              for (int ks = 0; ks < BK / 8; ks++) {
                const uint64_t ko = (uint64_t)(ks * 2);
                const uint64_t kob = B_MN ? (uint64_t)(ks * 64) : ko;
                tc2_mma_tf32(tmem_d, alo + ko, bhi + kob, idesc, (first && ks == 0) ? 0u : 1u);
                tc2_mma_tf32(tmem_d, ahi + ko, blo + kob, idesc, 1u);
                tc2_mma_tf32(tmem_d, ahi + ko, bhi + kob, idesc, 1u);
              }
              tc2_commit_both(empty0 + 8 * stage);
              if (++stage == P2_STAGES) {
                stage = 0;
                phase ^= 1;
              }
            }
            if (ok) tc2_commit_both(accf0 + 8 * buf);
          }
        }
      }
    }
  } else {
    // --------------------------------------------------- drain warps (both CTAs)
    asm volatile("setmaxnreg.inc.sync.aligned.u32 232;");
    const int ew = warp - FIRST_EPI_WARP;
    const int quarter = warp & 3;
    const int half = ew >> 2;
    const uint32_t leader_acce0 = map_to_cta(acce0, 0);
    TileCursor cur;
    int64_t cc = 0;
    bool ok = true;
    for (int64_t it = A_UPPER ? 0 : pair; p2_more<A_UPPER>(sp, it, pair, npairs, total) && ok;
         it += A_UPPER ? 1 : npairs) {
      const int64_t t = p2_tile<A_UPPER>(sp, tiles, it, pair, npairs, total);
      if (A_UPPER && t < 0) continue;
      int64_t tm2, tn;
      cur.seek(tiles, t, &tm2, &tn);
      const int64_t nchunks =
          (nkb - (A_UPPER ? tiles.first_kblock(tm2) : 0) + chunk_kblocks - 1) / chunk_kblocks;
      const int64_t r_base = tm2 * 256 + rank * 128 + quarter * 32;
      const int64_t cb = tn * PN + half * COLS;
      float acc[COLS];
#pragma unroll
      for (int i = 0; i < COLS; i++) acc[i] = 0.0f;
      if (beta != 0.0f && r_base + lane < M) {
#pragma unroll
        for (int q = 0; q < COLS / 32; q++)
          if (cb + q * 32 < N)
            asm volatile("prefetch.global.L2 [%0];" ::"l"(C + (r_base + lane) * ldc + cb + q * 32));
      }
      for (int64_t ch = 0; ch < nchunks && ok; ch++, cc++) {
        const uint32_t buf = (uint32_t)(cc & 1);
        const uint32_t use = (uint32_t)((cc >> 1) & 1);
        if (!mbar_wait_backoff(accf0 + 8 * buf, use)) {
          if (lane == 0) report_status(status, 34, (int32_t)blockIdx.x);
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t taddr =
            tmem_base + ((uint32_t)(quarter * 32) << 16) + buf * PN + (uint32_t)(half * COLS);
#pragma unroll
        for (int j = 0; j < COLS / 32; j += 2) {
          uint32_t v0[32], v1[32];
          tc_ld32(taddr + j * 32, v0);
          tc_ld32(taddr + j * 32 + 32, v1);
          tc_wait_ld();
#pragma unroll
          for (int i = 0; i < 32; i++) acc[j * 32 + i] += __uint_as_float(v0[i]);
#pragma unroll
          for (int i = 0; i < 32; i++) acc[j * 32 + 32 + i] += __uint_as_float(v1[i]);
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(leader_acce0 + 8 * buf);
      }
      if (!ok) break;
      epilogue_store<COLS>(acc, epi_stage[ew], lane, r_base, cb, M, N, ldc, C, alpha, beta,
                          tiles.lower != 0, tiles.row0);
    }
  }

  // Nobody leaves while the peer may still signal one of its barriers or use
  // the paired tensor memory.
  tc_fence_before();
  cluster_sync_all();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                 "r"(TMEM_COLS)
                 : "memory");
  }
}

// ===========================================================================
// Fused kernel for products with few tiles (configs such as 1024^3): ONE launch,
// no scratch memory.
//
//  * The lo parts are made inside the kernel.  TMA brings the raw fp32 tiles of
//    A and B into the ring; two "split" warps read each raw tile from shared
//    memory and write lo = tf32(x - trunc_tf32(x)) at the same offset of a
//    second buffer, so the (swizzled) layout of the lo tile equals that of the
//    raw tile by construction and no layout arithmetic is involved.  The tensor
//    core reads the raw tile as the hi part (it drops the low mantissa bits
//    itself).  The MMA thread waits on a "ready" barrier the split warps signal
//    after a generic->async proxy fence.
//  * Split-K inside a thread-block cluster.  The S CTAs of a cluster (S = 1, 2
//    or 4) share one 128x256 tile and take consecutive K ranges.  The partial
//    tiles are exchanged as a reduce-scatter: CTA q writes column slice r of its
//    partial tile to a small exchange buffer in global memory (it stays in L2),
//    ONE cluster barrier (release / acquire) orders the writes before the reads,
//    and CTA r adds the S slices of its column range in rank order - its own
//    from registers - so the sum does not depend on timing; then alpha/beta and
//    the store of its slice of C.  No counters, nothing to zero, no second
//    launch, and beta == 0 still never reads C.  (Distributed shared memory was
//    tried for the exchange, pulling and pushing: the SM-to-SM path moved the
//    96 KiB per CTA at ~20 bytes per cycle, 5-6 thousand cycles; through L2 the
//    same exchange takes about half of that.)
//
// One (tile, K range) per CTA; grid = tiles * S, cluster = (S, 1, 1).
// ===========================================================================
// lo = tf32(x - trunc_tf32(x)), rounded to nearest with ties away from zero like
// cvt.rna.tf32.f32 - done on the integer pipe (add half an ulp of TF32 to the
// magnitude, clear the 13 low bits): the conversion instruction runs at a
// fraction of the ALU rate, and this sits on the critical path of every K-block.
// lo = tf32(x - trunc_tf32(x)), rounded to nearest with ties away from zero like
// cvt.rna.tf32.f32 - done on the integer pipe (add half an ulp of TF32 to the
// magnitude, clear the 13 low bits): the conversion instruction runs at a
// fraction of the ALU rate, and this sits on the critical path of every K-block.
__device__ __forceinline__ void st_cluster_f4(uint32_t cluster_addr, float a, float b, float c,
                                              float d) {
  asm volatile("st.shared::cluster.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(cluster_addr), "f"(a),
               "f"(b), "f"(c), "f"(d)
               : "memory");
}
__device__ __forceinline__ float lo_part(float x) {
  const float hi = __uint_as_float(__float_as_uint(x) & 0xFFFFE000u);
  return __uint_as_float((__float_as_uint(x - hi) + 0x1000u) & 0xFFFFE000u);
}

#ifdef PGB200_FUSED_TRACE
// Development aid (not part of the product build): cycle stamps of a few CTAs.
__device__ long long g_fused_trace[8][16];
#define FUSED_STAMP(point)                                                        \
  do {                                                                            \
    if ((blockIdx.x & 15) == 0 && (blockIdx.x >> 4) < 8)                          \
      g_fused_trace[blockIdx.x >> 4][(point)] = clock64();                        \
  } while (0)
#else
#define FUSED_STAMP(point) \
  do {                     \
  } while (0)
#endif

template <bool B_MN, int S>
__global__ void __launch_bounds__(THREADS, 1)
tf32x3_gemm_fused_kernel(const __grid_constant__ CUtensorMap mapA,
                         const __grid_constant__ CUtensorMap mapB, int64_t M, int64_t N, int64_t K,
                         float alpha, float beta, float *__restrict__ C, int64_t ldc, Tiles tiles,
                         int chunk_kblocks, int b_blocked, int32_t *status) {
  static_assert(S == 1 || S == 2 || S == 4, "cluster size");
  constexpr int W = 128 / S;  // columns of the final tile each drain thread reduces and stores
  // Two rings share the 192 KiB: raw tiles (A 8 KiB + B 16 KiB per K-block), six
  // deep so that TMA runs ~4600 tensor-core cycles ahead (the first touch of
  // every panel comes from DRAM), and lo tiles, two deep: they are made just in
  // time and consumed at once.
  constexpr int RAW_BYTES = A_BYTES + B_BYTES;  // 24 KiB
  constexpr int RSTAGES = 6, LSTAGES = 2;
  static_assert((RSTAGES + LSTAGES) * RAW_BYTES + 1024 <= SMEM_BYTES, "ring does not fit");
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t bars[2 * RSTAGES + 2 * LSTAGES + 4];
  __shared__ uint32_t tmem_slot;
  __shared__ float epi_stage[EPI_WARPS][32][33];
  const uint32_t ring = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t *ring_ptr = smem_raw + (ring - smem_u32(smem_raw));
  const uint32_t lo_ring = ring + RSTAGES * RAW_BYTES;
  uint8_t *lo_ptr = ring_ptr + RSTAGES * RAW_BYTES;
  const uint32_t full0 = smem_u32(&bars[0]), empty0 = smem_u32(&bars[RSTAGES]);
  const uint32_t ready0 = smem_u32(&bars[2 * RSTAGES]);           // lo slot filled
  const uint32_t lfree0 = smem_u32(&bars[2 * RSTAGES + LSTAGES]);  // lo slot consumed
  const uint32_t accf0 = smem_u32(&bars[2 * RSTAGES + 2 * LSTAGES]);
  const uint32_t acce0 = smem_u32(&bars[2 * RSTAGES + 2 * LSTAGES + 2]);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = S > 1 ? cluster_ctarank() : 0u;
  if (threadIdx.x == 0) FUSED_STAMP(0);

  if (threadIdx.x == 64) {
    prefetch_tensor_map(&mapA);
    prefetch_tensor_map(&mapB);
  }
  if (threadIdx.x == 0) {
    for (int s = 0; s < RSTAGES; s++) {
      mbar_init(full0 + 8 * s, 1);
      mbar_init(empty0 + 8 * s, 1);
    }
    for (int s = 0; s < LSTAGES; s++) {
      mbar_init(ready0 + 8 * s, EPI_WARPS);  // one arrival per drain warp (they make the lo tiles)
      mbar_init(lfree0 + 8 * s, 1);
    }
    for (int b = 0; b < 2; b++) {
      mbar_init(accf0 + 8 * b, 1);
      mbar_init(acce0 + 8 * b, EPI_WARPS);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  // This CTA's work item: tile (cluster index), K-block range (rank).  32-bit
  // arithmetic where the values allow it: 64-bit divisions cost hundreds of
  // cycles each and sit in front of the first load.
  const int64_t t = (int64_t)(blockIdx.x / (unsigned)S);
  const int64_t nkb = (K + BK - 1) / BK;
  const int64_t kb_lo = (int64_t)rank * tiles.kper < nkb ? (int64_t)rank * tiles.kper : nkb;
  const int64_t kb_hi = kb_lo + tiles.kper < nkb ? kb_lo + tiles.kper : nkb;
  const int64_t nch =
      (int64_t)(((unsigned)(kb_hi - kb_lo) + (unsigned)chunk_kblocks - 1u) / (unsigned)chunk_kblocks);
  int64_t tm, tn;
  if (!tiles.lower) {
    // TileCursor::seek for a full product, on unsigned ints.
    const unsigned idx = (unsigned)t, tmn = (unsigned)tiles.tiles_m, tnn = (unsigned)tiles.tiles_n;
    const unsigned G = tiles.band > 0 ? (unsigned)tiles.band : (unsigned)TileCursor::G_DEFAULT;
    const unsigned per_group = G * tnn, grp = idx / per_group;
    const unsigned first = grp * G;
    const unsigned rows = tmn - first < G ? tmn - first : G;
    const unsigned in = idx - grp * per_group;
    tm = first + in % rows;
    tn = in / rows;
  } else {
    TileCursor cur;
    cur.seek(tiles, t, &tm, &tn);
  }
  // The producer's state lives across the CTA-wide sync below: its first loads
  // (cold: DRAM and page-table latency) leave before tensor memory is allocated.
  uint32_t p_stage = 0, p_phase = 0;
  int64_t p_kb = kb_lo;
  auto produce = [&](int64_t kb) {
    const uint32_t dst = ring + p_stage * RAW_BYTES;
    const uint32_t bar = full0 + 8 * p_stage;
    mbar_expect_tx(bar, RAW_BYTES);
    const int k0 = (int)(kb * BK);
    tma_load_2d(dst, &mapA, bar, k0, (int)(tm * BM));
    if (B_MN) {
      // Row-major B as it lies: eight [BK x 32] column blocks, by one 3-D copy
      // when N is a multiple of 32, else by eight 2-D copies (zero-filled past
      // column N).
      if (b_blocked) {
        tma_load_3d(dst + A_BYTES, &mapB, bar, 0, k0, (int)(tn * (BN / 32)));
      } else {
#pragma unroll
        for (int j = 0; j < BN / 32; j++)
          tma_load_2d(dst + A_BYTES + j * (BK * 128), &mapB, bar, (int)(tn * BN) + 32 * j, k0);
      }
    } else {
      tma_load_2d(dst + A_BYTES, &mapB, bar, k0, (int)(tn * BN));
    }
    if (++p_stage == RSTAGES) {
      p_stage = 0;
      p_phase ^= 1;
    }
  };
  if (threadIdx.x == 0) {
    // Every stage is free at the start: fill the ring (thread 0 initialised the
    // barriers itself, so it may use them before the sync).
    for (; p_kb < kb_hi && p_kb < kb_lo + RSTAGES; p_kb++) {
      if (p_kb == kb_lo) FUSED_STAMP(2);
      produce(p_kb);
    }
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     smem_u32(&tmem_slot)),
                 "r"(TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_slot;
  if (threadIdx.x == 0) FUSED_STAMP(1);

  if (warp < FIRST_EPI_WARP) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 40;");
    if (warp == 0) {
      // ------------------------------------------------------------ TMA producer
      if (lane == 0) {
        for (; p_kb < kb_hi; p_kb++) {
          if (!mbar_wait(empty0 + 8 * p_stage, p_phase ^ 1)) {
            report_status(status, 41, (int32_t)blockIdx.x);
            break;
          }
          produce(p_kb);
        }
      }
    } else if (warp == 1) {
      // -------------------------------------------------------------- MMA issuer
      if (lane == 0) {
        uint32_t stage = 0, lslot = 0, lphase = 0;
        bool ok = true;
        for (int64_t ch = 0; ch < nch && ok; ch++) {
          const uint32_t buf = (uint32_t)(ch & 1);
          const uint32_t use = (uint32_t)((ch >> 1) & 1);
          if (!mbar_wait(acce0 + 8 * buf, use ^ 1)) {
            report_status(status, 42, (int32_t)blockIdx.x);
            break;
          }
          tc_fence_after();
          const uint32_t tmem_d = tmem_base + buf * BN;
          const int64_t kb_first = kb_lo + ch * chunk_kblocks;
          const int64_t kb_end = kb_first + chunk_kblocks < kb_hi ? kb_first + chunk_kblocks : kb_hi;
          for (int64_t kb = kb_first; kb < kb_end; kb++) {
            // The lo tile is made from the raw tile, so "lo ready" implies "raw full".
            if (!mbar_wait(ready0 + 8 * lslot, lphase)) {
              report_status(status, 43, (int32_t)blockIdx.x);
              ok = false;
              break;
            }
            tc_fence_after();
            if (kb == kb_lo) FUSED_STAMP(4);
            const uint32_t sr = ring + stage * RAW_BYTES, sl = lo_ring + lslot * RAW_BYTES;
            const uint64_t ahi = smem_desc_sw64(sr), alo = smem_desc_sw64(sl);
            const uint64_t bhi = B_MN ? smem_desc_mn_sw128(sr + A_BYTES) : smem_desc_sw64(sr + A_BYTES);
            const uint64_t blo = B_MN ? smem_desc_mn_sw128(sl + A_BYTES) : smem_desc_sw64(sl + A_BYTES);
            constexpr uint32_t idesc = B_MN ? IDESC_BMN : IDESC;
            const bool first = (kb == kb_first);
#pragma unroll
            for (int ks = 0; ks < BK / 8; ks++) {
              const uint64_t ko = (uint64_t)(ks * 2);
              const uint64_t kob = B_MN ? (uint64_t)(ks * 64) : ko;
              tc_mma_tf32(tmem_d, alo + ko, bhi + kob, idesc, (first && ks == 0) ? 0u : 1u);
              tc_mma_tf32(tmem_d, ahi + ko, blo + kob, idesc, 1u);
              tc_mma_tf32(tmem_d, ahi + ko, bhi + kob, idesc, 1u);
            }
            tc_commit(empty0 + 8 * stage);   // raw stage back to the producer
            tc_commit(lfree0 + 8 * lslot);   // lo slot back to the drain warps
            if (++stage == RSTAGES) stage = 0;
            if (++lslot == LSTAGES) {
              lslot = 0;
              lphase ^= 1;
            }
          }
          if (ok) tc_commit(accf0 + 8 * buf);
        }
        FUSED_STAMP(5);
      }
    }
    if (S > 1) {
      // The cluster barrier of the drain warps' reduction, matched here.
      __syncwarp();
      cluster_sync_all();
    }
  } else {
    // ------------------------------------------------------------- drain warps
    asm volatile("setmaxnreg.inc.sync.aligned.u32 232;");
    const int quarter = warp & 3;
    const int half = (warp - FIRST_EPI_WARP) >> 2;
    bool ok = true;
    float acc[128];
#pragma unroll
    for (int i = 0; i < 128; i++) acc[i] = 0.0f;
    if (beta != 0.0f) {
      // This thread's slice of C towards L2 while the tensor cores work.
      const int64_t pr = tm * BM + quarter * 32 + lane, pc = tn * BN + half * 128 + rank * W;
      if (pr < M) {
#pragma unroll
        for (int q = 0; q < W / 32; q++)
          if (pc + q * 32 < N)
            asm volatile("prefetch.global.L2 [%0];" ::"l"(C + pr * ldc + pc + q * 32));
      }
    }
    // Adds accumulator chunk `ch` (tensor memory) into the registers.
    auto drain_chunk = [&](int64_t ch) -> bool {
      const uint32_t buf = (uint32_t)(ch & 1);
      const uint32_t use = (uint32_t)((ch >> 1) & 1);
      if (!mbar_wait_backoff(accf0 + 8 * buf, use)) {
        if (lane == 0) report_status(status, 44, (int32_t)blockIdx.x);
        return false;
      }
      tc_fence_after();
      const uint32_t taddr =
          tmem_base + ((uint32_t)(quarter * 32) << 16) + buf * BN + (uint32_t)(half * 128);
#pragma unroll
      for (int j = 0; j < 4; j += 2) {
        uint32_t v0[32], v1[32];
        tc_ld32(taddr + j * 32, v0);
        tc_ld32(taddr + j * 32 + 32, v1);
        tc_wait_ld();
#pragma unroll
        for (int i = 0; i < 32; i++) acc[j * 32 + i] += __uint_as_float(v0[i]);
#pragma unroll
        for (int i = 0; i < 32; i++) acc[j * 32 + 32 + i] += __uint_as_float(v1[i]);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(acce0 + 8 * buf);
      return true;
    };
    // The 256 drain threads also make the lo tiles (6 float4 each per K-block:
    // two spare warps alone took longer per K-block than its MMAs).  A chunk's
    // accumulator is drained once a later lo slot has come back, which shows that
    // the chunk's last MMA has retired; the MMA thread then still has up to two
    // K-blocks in hand while the drain runs.
    const int dtid = (int)threadIdx.x - 32 * FIRST_EPI_WARP;  // 0..255
    const int64_t lag = chunk_kblocks > 1 ? 1 : 0;
    int64_t drained = 0;
    {
      uint32_t stage = 0, phase = 0, lslot = 0, lphase = 0;
      for (int64_t kb = kb_lo; kb < kb_hi && ok; kb++) {
        if (!mbar_wait(full0 + 8 * stage, phase) || !mbar_wait(lfree0 + 8 * lslot, lphase ^ 1)) {
          if (lane == 0) report_status(status, 45, (int32_t)blockIdx.x);
          ok = false;
          break;
        }
        if (kb == kb_lo && dtid == 0) FUSED_STAMP(3);
        const float4 *raw = reinterpret_cast<const float4 *>(ring_ptr + stage * RAW_BYTES);
        float4 *lo = reinterpret_cast<float4 *>(lo_ptr + lslot * RAW_BYTES);
        float4 x[RAW_BYTES / 16 / 256];
#pragma unroll
        for (int i = 0; i < RAW_BYTES / 16 / 256; i++) x[i] = raw[dtid + 256 * i];
#pragma unroll
        for (int i = 0; i < RAW_BYTES / 16 / 256; i++)
          lo[dtid + 256 * i] =
              make_float4(lo_part(x[i].x), lo_part(x[i].y), lo_part(x[i].z), lo_part(x[i].w));
        // Make the generic-proxy writes visible to the tensor core's reads.
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncwarp();
        if (lane == 0) mbar_arrive(ready0 + 8 * lslot);
        if (++stage == RSTAGES) {
          stage = 0;
          phase ^= 1;
        }
        if (++lslot == LSTAGES) {
          lslot = 0;
          lphase ^= 1;
        }
        while (ok && drained + 1 < nch && kb - kb_lo >= (drained + 1) * chunk_kblocks + lag)
          ok = drain_chunk(drained++);
      }
    }
    while (ok && drained < nch) ok = drain_chunk(drained++);
    if (dtid == 0) FUSED_STAMP(6);

    const int ew = warp - FIRST_EPI_WARP;
    const int64_t r_base = tm * BM + quarter * 32;
    const int64_t cb = tn * BN + half * 128;
    if (S == 1) {
      if (ok)
        epilogue_store<128>(acc, epi_stage[ew], lane, r_base, cb, M, N, ldc, C, alpha, beta,
                            tiles.lower != 0, tiles.row0);
    } else {
      // Reduce-scatter through the exchange buffer: slice r of this CTA's
      // partial tile goes to block (cluster, receiver r, source rank) as
      // [float4 index in the slice][drain thread], so every warp access is 512
      // contiguous bytes; the own slice stays in registers.
      const int dt = (int)threadIdx.x - 32 * FIRST_EPI_WARP;  // drain thread 0..255
      constexpr int SLICE4 = W / 4;                            // float4 per thread and slice
      float4 *xbuf = reinterpret_cast<float4 *>(tiles.partial) +
                     (size_t)t * S * S * SLICE4 * 256;
      if (dt == 0) FUSED_STAMP(7);
#pragma unroll
      for (int j = 0; j < 32; j++) {
        const uint32_t r = (uint32_t)(j / SLICE4), jl = (uint32_t)(j % SLICE4);
        if (r != rank)
          __stcg(xbuf + ((size_t)(r * S + rank) * SLICE4 + jl) * 256 + dt,
                 make_float4(acc[4 * j], acc[4 * j + 1], acc[4 * j + 2], acc[4 * j + 3]));
      }
      // Own slice: `acc` is indexed with a run-time rank, so it is selected with
      // constant indices (the array stays in registers and is dead afterwards).
      float mine[W];
#pragma unroll
      for (int rr = 0; rr < S; rr++)
        if ((uint32_t)rr == rank) {
#pragma unroll
          for (int i = 0; i < W; i++) mine[i] = acc[rr * W + i];
        }
      // The old values of this CTA's slice of C, asked for before the barrier so
      // that their latency hides behind it (interior tiles only; edge and
      // diagonal tiles take the general epilogue below).
      const int64_t cs = cb + rank * W;  // first column of this thread block's slice
      const bool interior = (r_base + 31 < M) && (cs + W - 1 < N) &&
                            (!tiles.lower || cs + W - 1 <= r_base + tiles.row0);
      float cold[W];
      if (interior && beta != 0.0f) {
#pragma unroll
        for (int b = 0; b < W / 32; b++)
#pragma unroll
          for (int q = 0; q < 32; q++)
            cold[b * 32 + q] = __ldcs(C + (r_base + q) * ldc + cs + b * 32 + lane);
      }
      __syncwarp();
      if (dt == 0) FUSED_STAMP(8);
      cluster_sync_all();  // every peer's slices are written (release) and visible (acquire)
      if (dt == 0) FUSED_STAMP(9);
      float red[W];
#pragma unroll
      for (int q = 0; q < S; q++) {
#pragma unroll
        for (int j = 0; j < SLICE4; j++) {
          float4 v;
          if ((uint32_t)q == rank)
            v = make_float4(mine[4 * j], mine[4 * j + 1], mine[4 * j + 2], mine[4 * j + 3]);
          else
            v = __ldcg(xbuf + ((size_t)(rank * S + q) * SLICE4 + j) * 256 + dt);
          if (q == 0) {
            red[4 * j] = v.x; red[4 * j + 1] = v.y; red[4 * j + 2] = v.z; red[4 * j + 3] = v.w;
          } else {
            red[4 * j] += v.x; red[4 * j + 1] += v.y; red[4 * j + 2] += v.z; red[4 * j + 3] += v.w;
          }
        }
      }
      if (dt == 0) FUSED_STAMP(10);
      if (ok && interior) {
        // Turn each 32x32 block through the padded shared tile so that C is
        // written as full 128-byte row segments (lane = column).
        float(*stg)[33] = epi_stage[ew];
#pragma unroll
        for (int b = 0; b < W / 32; b++) {
          __syncwarp();
#pragma unroll
          for (int i = 0; i < 32; i++) stg[lane][i] = alpha * red[b * 32 + i];
          __syncwarp();
#pragma unroll
          for (int q = 0; q < 32; q++) {
            const float o = stg[q][lane];
            C[(r_base + q) * ldc + cs + b * 32 + lane] =
                (beta != 0.0f) ? fmaf(beta, cold[b * 32 + q], o) : o;
          }
        }
      } else if (ok) {
        epilogue_store<W>(red, epi_stage[ew], lane, r_base, cs, M, N, ldc, C, alpha, beta,
                          tiles.lower != 0, tiles.row0);
      }
      if (dt == 0) FUSED_STAMP(11);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                 "r"(TMEM_COLS)
                 : "memory");
  }
  if (threadIdx.x == 32) FUSED_STAMP(12);
}

}  // namespace

#ifdef PGB200_FUSED_TRACE
extern "C" int32_t pgb200DebugFusedTrace(long long *out) {
  return cudaMemcpyFromSymbol(out, g_fused_trace, sizeof(g_fused_trace)) == cudaSuccess ? 0 : 2;
}
#endif

// Self-test of the bounded-wait machinery: one CTA waits on an mbarrier that
// nothing ever arrives at, with a caller-chosen cycle limit, and must come back
// with a status code instead of hanging.
__global__ void wait_timeout_selftest_kernel(long long limit_cycles, int32_t *status) {
  __shared__ __align__(8) uint64_t bar;
  if (threadIdx.x == 0) {
    mbar_init(smem_u32(&bar), 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    const long long t0 = clock64();
    bool done = false;
    while (!done && clock64() - t0 <= limit_cycles) done = mbar_try(smem_u32(&bar), 0);
    if (!done) report_status(status, 99, (int32_t)blockIdx.x);
  }
}

int32_t wait_timeout_selftest(cudaStream_t s, long long limit_cycles) {
  Runtime *rt = nullptr;
  PGB_TRY(get_runtime(&rt));
  if (limit_cycles < 0) limit_cycles = 0;
  if (limit_cycles > 2000000000ll) limit_cycles = 2000000000ll;  // never more than ~1 s
  wait_timeout_selftest_kernel<<<1, 32, 0, s>>>(limit_cycles, rt->status_dev);
  note_launch(PATH_TCGEN05);
  PGB_CUDA(cudaGetLastError());
  return PGB200_OK;
}

int32_t tf32_peak_probe(cudaStream_t s, double *gflops) {
  Runtime *rt = nullptr;
  PGB_TRY(get_runtime(&rt));
  const int iters = 8192, smem = A_BYTES + B_BYTES + 1024;
  PGB_CUDA(cudaFuncSetAttribute(tf32_probe_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                smem));
  cudaEvent_t e0, e1;
  PGB_CUDA(cudaEventCreate(&e0));
  PGB_CUDA(cudaEventCreate(&e1));
  float best = 1e30f;
  for (int r = 0; r < 5; r++) {
    PGB_CUDA(cudaEventRecord(e0, s));
    tf32_probe_kernel<<<rt->num_sms, 128, smem, s>>>(iters, rt->status_dev);
    PGB_CUDA(cudaEventRecord(e1, s));
    PGB_CUDA(cudaEventSynchronize(e1));
    float ms = 0;
    PGB_CUDA(cudaEventElapsedTime(&ms, e0, e1));
    if (r >= 1 && ms < best) best = ms;
  }
  cudaEventDestroy(e0);
  cudaEventDestroy(e1);
  PGB_CUDA(cudaGetLastError());
  *gflops = 2.0 * BM * BN * 8 * (double)iters * rt->num_sms / (best * 1e-3) * 1e-9;
  return PGB200_OK;
}

int32_t tf32x3_gemm(cudaStream_t s, int64_t M, int64_t N, int64_t K, float alpha, const float *A,
                    int64_t lda, const float *B, int64_t ldb, bool transB, float beta, float *C,
                    int64_t ldc, bool lower, int64_t row0, bool a_upper) {
  Runtime *rt = nullptr;
  PGB_TRY(get_runtime(&rt));
  if (K == 0) return PGB200_ERR_UNSUPPORTED;  // nothing to contract: SIMT path scales C
  if (M >= (int64_t(1) << 31) || N >= (int64_t(1) << 31) || K >= (int64_t(1) << 31))
    return PGB200_ERR_UNSUPPORTED;
  const int64_t Kp = (K + 31) / 32 * 32, Np = (N + 31) / 32 * 32;
  const bool planes_only = rt->cfg.sgemm_planes_only != 0;  // never use operands in place
  // An operand whose rows are 16-byte aligned is used in place as its own "hi"
  // plane (the tensor core truncates fp32 to TF32); only its "lo" plane is
  // written.  Otherwise both planes are written (and B is transposed).
  const bool a_raw = !planes_only && aligned16(A) && (lda % 4) == 0;
  const bool b_raw = !planes_only && aligned16(B) && (ldb % 4) == 0;
  // For the rank-k update both operands are rows of one matrix: when A's rows
  // are a sub-range of B's rows the A planes are views into the B planes.
  const bool shared_planes = transB && (ldb == lda) && (B <= A) && ((A - B) % lda == 0) &&
                             ((A - B) / lda + M <= N);
  const int64_t a_off_rows = shared_planes ? (A - B) / lda : 0;
  // A row-major B can be consumed as it lies (N-major operand), which saves the
  // transposing pre-pass, but the tensor cores run the N-major 32-byte-atom
  // layout several percent slower (measured: 398 vs 372 ms at 32768^3).  The
  // pre-pass is paid once per call, the slowdown per row of A: for tall
  // products transpose B once, otherwise use it in place.
  const bool b_mn = !transB && b_raw && (M < 12288 || rt->cfg.sgemm_b_in_place);

  // Tile width: 256 columns normally.  When 256-wide tiles would leave more
  // than half of the SMs without a tile, either the K range of every tile is
  // split over several CTAs (each keeps the full-rate N = 256 MMA shape; an
  // M128 MMA takes 128 cycles whatever its N, so narrow tiles waste the tensor
  // core) or, when K is too short for that, 64-column tiles are used.
  const int chunk =
      rt->cfg.sgemm_chunk_kblocks > 0 ? rt->cfg.sgemm_chunk_kblocks : DEFAULT_CHUNK_KBLOCKS;
  const int64_t tiles256 = ((M + BM - 1) / BM) * ((N + 255) / 256);
  const int64_t nkb_all = (K + BK - 1) / BK;
  int bn = (tiles256 * 2 <= rt->num_sms) ? 64 : 256;
  int splits = 1;
  int64_t kper = nkb_all;
  if (bn == 64 && !rt->cfg.no_split_k) {
    int64_t sp = rt->num_sms / tiles256;       // CTAs available per tile
    const int64_t by_k = nkb_all / (2 * chunk);  // at least two chunks per split
    if (sp > by_k) sp = by_k;
    if (sp > MAX_SPLITS) sp = MAX_SPLITS;
    if (sp >= 2) {
      kper = ((nkb_all + sp - 1) / sp + chunk - 1) / chunk * chunk;
      splits = (int)((nkb_all + kper - 1) / kper);
      if (splits >= 2)
        bn = 256;
      else
        splits = 1;
    }
  }
  // Few tiles and both operands usable in place: the fused kernel - lo parts
  // made in shared memory, K split inside a cluster, one launch, no scratch.
  if (tiles256 * 2 <= rt->num_sms && a_raw && b_raw) {
    Tiles ft = {};
    ft.tiles_m = (M + BM - 1) / BM;
    ft.tiles_n = (N + 255) / 256;
    ft.bn = 256;
    ft.bm = BM;
    ft.row0 = row0;
    ft.lower = lower ? 1 : 0;
    ft.total = count_tiles(ft);
    int S = 1;
    if (!rt->cfg.no_split_k && ft.total > 0) {
      int64_t sp = rt->num_sms / ft.total;         // CTAs available per tile
      const int64_t by_k = nkb_all / (2 * chunk);  // at least two chunks per K range
      if (sp > by_k) sp = by_k;
      S = sp >= 4 ? 4 : (sp >= 2 ? 2 : 1);
    }
    int64_t fk = ((nkb_all + S - 1) / S + chunk - 1) / chunk * chunk;
    while (S > 1 && (int64_t)(S - 1) * fk >= nkb_all) {  // a rank would get no K-block
      S >>= 1;
      fk = ((nkb_all + S - 1) / S + chunk - 1) / chunk * chunk;
    }
    ft.splits = S;
    ft.kper = fk;
    // Exchange buffer of the in-cluster reduce-scatter: S x S slices per tile,
    // S * 128 KiB in all per tile; written and read once, it lives in L2.
    PoolBuffer xchg;
    if (S > 1) {
      PGB_CUDA(xchg.alloc((size_t)ft.total * S * BM * 256 * sizeof(float), s));
      ft.partial = xchg.as<float>();
    }
    CUtensorMap mA, mB;
    const int fb_blocked = (!transB && (N % 32) == 0) ? 1 : 0;
    PGB_TRY(make_plane_map(&mA, A, M, K, lda, BM));
    if (transB)
      PGB_TRY(make_plane_map(&mB, B, N, K, ldb, 256));
    else if (fb_blocked)
      PGB_TRY(make_nmajor_map_blocked(&mB, B, K, N, ldb, 256));
    else
      PGB_TRY(make_nmajor_map(&mB, B, K, N, ldb));
    cudaLaunchConfig_t lc = {};
    lc.gridDim = dim3((unsigned)(ft.total * S), 1, 1);
    lc.blockDim = dim3(THREADS, 1, 1);
    lc.dynamicSmemBytes = SMEM_BYTES;
    lc.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = (unsigned)S;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    lc.attrs = attr;
    lc.numAttrs = S > 1 ? 1 : 0;
    auto launchf = [&](auto kernel) -> int32_t {
      PGB_TRY(ensure_dynamic_smem((const void *)kernel, SMEM_BYTES));
      PGB_CUDA(cudaLaunchKernelEx(&lc, kernel, mA, mB, M, N, K, alpha, beta, C, ldc, ft, chunk,
                                  fb_blocked, rt->status_dev));
      return PGB200_OK;
    };
    if (transB) {
      PGB_TRY(S == 4   ? launchf(tf32x3_gemm_fused_kernel<false, 4>)
              : S == 2 ? launchf(tf32x3_gemm_fused_kernel<false, 2>)
                       : launchf(tf32x3_gemm_fused_kernel<false, 1>));
    } else {
      PGB_TRY(S == 4   ? launchf(tf32x3_gemm_fused_kernel<true, 4>)
              : S == 2 ? launchf(tf32x3_gemm_fused_kernel<true, 2>)
                       : launchf(tf32x3_gemm_fused_kernel<true, 1>));
    }
    note_launch(PATH_TCGEN05);
    return PGB200_OK;
  }
  const int64_t ldp = (N + 3) / 4 * 4;
  const size_t part_n = splits > 1 ? (size_t)splits * M * ldp : 0;

  // Scratch layout (floats): [B lo][B hi?][A lo?][A hi?][split-K partials?]
  const size_t b_lo_n = b_mn ? (size_t)K * Np : (size_t)N * Kp;
  const bool b_inplace = b_mn || (transB && b_raw);  // B serves as its own hi part
  const size_t b_hi_n = b_inplace ? 0 : (size_t)N * Kp;
  const size_t a_lo_n = shared_planes ? 0 : (size_t)M * Kp;
  const size_t a_hi_n = (shared_planes || a_raw) ? 0 : (size_t)M * Kp;
  PoolBuffer scratch;  // this call's own planes and partial products, released in stream order
  const size_t ctr_n = 64;  // the two-CTA kernel's round counter, on a line of its own
  PGB_CUDA(scratch.alloc((b_lo_n + b_hi_n + a_lo_n + a_hi_n + part_n + ctr_n) * sizeof(float), s));
  void *ws = scratch.ptr;
  float *Blo = static_cast<float *>(ws);
  float *Bhi_pl = Blo + b_lo_n;
  float *Alo_pl = Bhi_pl + b_hi_n;
  float *Ahi_pl = Alo_pl + a_lo_n;
  float *partial = Ahi_pl + a_hi_n;
  int32_t *step_ctr = reinterpret_cast<int32_t *>(partial + part_n);

  const int64_t cap = (int64_t)rt->num_sms * 8;
  auto grid_for = [&](int64_t total) {
    int64_t g = (total + 255) / 256;
    return (unsigned)(g < 1 ? 1 : (g > cap ? cap : g));
  };
  // ---- B ----
  const float *Bhi = nullptr;
  int64_t bhi_ld = Kp;
  // Both operands usable in place: their lo planes come from one launch.
  const bool pair = b_inplace && a_raw && !shared_planes;
  if (pair) {
    const int64_t b_rows = b_mn ? K : N, b_cols = b_mn ? N : K, b_colsP = b_mn ? Np : Kp;
    const unsigned g0 = grid_for(b_rows * (b_colsP / 4)), g1 = grid_for(M * (Kp / 4));
    split_lo_pair_kernel<<<g0 + g1, 256, 0, s>>>(B, ldb, b_rows, b_cols, b_colsP, Blo, (int)g0, A,
                                                  lda, M, K, Kp, Alo_pl);
    Bhi = B;
    bhi_ld = ldb;
  } else if (b_mn) {
    split_lo_kernel<<<grid_for(K * (Np / 4)), 256, 0, s>>>(B, ldb, K, N, Np, Blo);
    Bhi = B;
    bhi_ld = ldb;
  } else if (transB && b_raw) {
    split_lo_kernel<<<grid_for(N * (Kp / 4)), 256, 0, s>>>(B, ldb, N, K, Kp, Blo);
    Bhi = B;
    bhi_ld = ldb;
  } else if (transB) {
    split_rows_kernel<<<grid_for(N * Kp), 256, 0, s>>>(B, ldb, N, K, Kp, Bhi_pl, Blo);
    Bhi = Bhi_pl;
  } else {
    const int64_t tk = Kp / 32, tn = (N + 31) / 32;
    PGB_REQUIRE(tk * tn < (int64_t(1) << 31), "tf32x3_gemm: operand too large");
    split_transpose_kernel<<<(unsigned)(tk * tn), 256, 0, s>>>(B, ldb, K, N, Kp, Bhi_pl, Blo, tk);
    Bhi = Bhi_pl;
  }
  note_launch(PATH_TCGEN05);
  // ---- A ----
  const float *Ahi = nullptr, *Alo = nullptr;
  int64_t ahi_ld = Kp;
  if (shared_planes) {
    Alo = Blo + a_off_rows * Kp;
    Ahi = Bhi + a_off_rows * bhi_ld;
    ahi_ld = bhi_ld;
  } else if (a_raw) {
    if (!pair) {
      split_lo_kernel<<<grid_for(M * (Kp / 4)), 256, 0, s>>>(A, lda, M, K, Kp, Alo_pl);
      note_launch(PATH_TCGEN05);
    }
    Alo = Alo_pl;
    Ahi = A;
    ahi_ld = lda;
  } else {
    split_rows_kernel<<<grid_for(M * Kp), 256, 0, s>>>(A, lda, M, K, Kp, Ahi_pl, Alo_pl);
    note_launch(PATH_TCGEN05);
    Alo = Alo_pl;
    Ahi = Ahi_pl;
  }
  PGB_CUDA(cudaGetLastError());

  CUtensorMap mAhi, mAlo, mBhi, mBlo;
  PGB_TRY(make_plane_map(&mAhi, Ahi, M, K, ahi_ld, BM));
  PGB_TRY(make_plane_map(&mAlo, Alo, M, K, Kp, BM));
  const bool bhi_blocked = b_mn && (N % 32) == 0;
  if (b_mn) {
    if (bhi_blocked)
      PGB_TRY(make_nmajor_map_blocked(&mBhi, Bhi, K, N, bhi_ld, bn));
    else
      PGB_TRY(make_nmajor_map(&mBhi, Bhi, K, N, bhi_ld));
    PGB_TRY(make_nmajor_map_blocked(&mBlo, Blo, K, Np, Np, bn));
  } else {
    PGB_TRY(make_plane_map(&mBhi, Bhi, N, K, bhi_ld, bn));
    PGB_TRY(make_plane_map(&mBlo, Blo, N, K, Kp, bn));
  }

  Tiles tiles;
  tiles.band = 0;
  tiles.step_ctr = nullptr;
  tiles.tiles_m = (M + BM - 1) / BM;
  tiles.tiles_n = (N + bn - 1) / bn;
  tiles.bn = bn;
  tiles.bm = BM;
  tiles.row0 = row0;
  tiles.lower = lower ? 1 : 0;
  tiles.a_upper = 0;  // a hint only the two-CTA kernel takes; the product is the same without it
  tiles.splits = splits;
  tiles.kper = kper;
  tiles.partial = partial;
  tiles.ldp = ldp;
  tiles.total = count_tiles(tiles);
  int64_t ctas = rt->num_sms - (rt->cfg.reserve_sms > 0 ? rt->cfg.reserve_sms : 0);
  if (ctas < 1) ctas = 1;
  const int64_t work = tiles.total * splits;
  const unsigned grid = (unsigned)(work < ctas ? work : ctas);
  // Meeting between rounds of tiles: measured (8192 x 8192 and 16384 x 16384
  // by K) it costs 3-5 % at K = 512, nothing at 1024-2048 and gains from there
  // on (16384 x 32768 x 2048: 7.74 vs 7.97 ms; 32768^3: 268 vs 319 ms).
  const bool meet_k = K >= 2048 && !rt->cfg.no_step_sync;
  // Large full products: the two-CTA kernel (256x256 tiles on SM pairs).
  // Measured against the one-CTA kernel: 8192^3 4.01-4.18 vs 4.45 ms, 16384^3
  // 36.7-38.1 vs 40.5-40.8 ms, 32768^3 354-356 vs 423-443 ms (same GPU, back to
  // back).  pgb200Config.no_two_cta switches it off.
  const int pn = 256;  // pair tile width (128 also works: measured slower than split-K where it applied)
  const bool two_cta = bn == 256 && splits == 1 && M >= 512 && (!b_mn || bhi_blocked) &&
                       !rt->cfg.no_two_cta;
  if (two_cta) {
    CUtensorMap m2Bhi, m2Blo;
    if (b_mn) {
      PGB_TRY(make_nmajor_map_blocked(&m2Bhi, Bhi, K, N, bhi_ld, pn / 2));
      PGB_TRY(make_nmajor_map_blocked(&m2Blo, Blo, K, Np, Np, pn / 2));
    } else {
      PGB_TRY(make_plane_map(&m2Bhi, Bhi, N, K, bhi_ld, pn / 2));
      PGB_TRY(make_plane_map(&m2Blo, Blo, N, K, Kp, pn / 2));
    }
    Tiles t2 = tiles;
    t2.bm = 256;
    t2.bn = pn;
    t2.tiles_m = (M + 255) / 256;
    t2.tiles_n = (N + pn - 1) / pn;
    t2.a_upper = (a_upper && !lower) ? 1 : 0;
    t2.total = count_tiles(t2);
    int64_t pairs = t2.total;
    const int64_t max_pairs = ctas / 2 > 0 ? ctas / 2 : 1;
    if (pairs > max_pairs) pairs = max_pairs;
    if (!t2.a_upper && t2.total > pairs && meet_k) {
      PGB_CUDA(cudaMemsetAsync(step_ctr, 0, sizeof(int32_t), s));
      t2.step_ctr = step_ctr;
    }
    cudaLaunchConfig_t lc = {};
    lc.gridDim = dim3((unsigned)(2 * pairs), 1, 1);
    lc.blockDim = dim3(THREADS, 1, 1);
    lc.dynamicSmemBytes = SMEM_BYTES;
    lc.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    lc.attrs = attr;
    lc.numAttrs = 1;
    auto launch2 = [&](auto kernel, const auto &sp) -> int32_t {
      PGB_TRY(ensure_dynamic_smem((const void *)kernel, SMEM_BYTES));
      PGB_CUDA(cudaLaunchKernelEx(&lc, kernel, mAhi, mAlo, m2Bhi, m2Blo, M, N, K, alpha, beta, C, ldc,
                                  t2, chunk, sp, rt->status_dev));
      return PGB200_OK;
    };
    if (t2.a_upper) {
      // Tiles differ in length: hand them out longest-first when the table fits
      // (same band walk as TileCursor::seek for a full product).
      SchedParam<true> sp;
      sp.use = 0;
      if (t2.total > pairs) {
        const int64_t nkb = (K + BK - 1) / BK;
        std::vector<int64_t> cost((size_t)t2.total);
        const int64_t G = t2.band > 0 ? t2.band : TileCursor::G_DEFAULT;
        const int64_t per_group = G * t2.tiles_n;
        for (int64_t t = 0; t < t2.total; t++) {
          const int64_t grp = t / per_group, first = grp * G;
          const int64_t rows =
              (t2.tiles_m - first < G) ? (t2.tiles_m - first) : G;
          const int64_t tm = first + (t - grp * per_group) % rows;
          const int64_t len = nkb - (tm * 256) / BK;
          cost[(size_t)t] = (len > 0 ? len : 0) + 1;
        }
        if (build_lpt_schedule(cost.data(), t2.total, (int)pairs, &sp.s)) sp.use = 1;
      }
      PGB_TRY(b_mn ? launch2(tf32x3_gemm_2cta_kernel<true, true, 256>, sp)
                   : launch2(tf32x3_gemm_2cta_kernel<false, true, 256>, sp));
    } else {
      const SchedParam<false> sp;
      PGB_TRY(b_mn ? launch2(tf32x3_gemm_2cta_kernel<true, false, 256>, sp)
                   : launch2(tf32x3_gemm_2cta_kernel<false, false, 256>, sp));
    }
    note_launch(PATH_TCGEN05);
    PGB_CUDA(cudaGetLastError());
    return PGB200_OK;
  }
  if (splits == 1 && tiles.total > (int64_t)grid && meet_k) {
    PGB_CUDA(cudaMemsetAsync(step_ctr, 0, sizeof(int32_t), s));
    tiles.step_ctr = step_ctr;
  }
  auto launch = [&](auto kernel, int bhi_blk) -> int32_t {
    PGB_TRY(ensure_dynamic_smem((const void *)kernel, SMEM_BYTES));
    kernel<<<grid, THREADS, SMEM_BYTES, s>>>(mAhi, mAlo, mBhi, mBlo, M, N, K, alpha, beta, C, ldc,
                                             tiles, chunk, bhi_blk, rt->status_dev);
    return PGB200_OK;
  };
  if (splits > 1) {
    PGB_TRY(b_mn ? launch(tf32x3_gemm_kernel<true, 256, true>, bhi_blocked ? 1 : 0)
                 : launch(tf32x3_gemm_kernel<false, 256, true>, 0));
    const int64_t items = M * (ldp / 4);
    splitk_reduce_kernel<<<(unsigned)((items + 127) / 128), 128, 0, s>>>(
        partial, ldp, splits, M, N, alpha, beta, C, ldc, lower ? 1 : 0, row0);
    note_launch(PATH_TCGEN05);
  } else if (b_mn) {
    PGB_TRY(bn == 256 ? launch(tf32x3_gemm_kernel<true, 256, false>, bhi_blocked ? 1 : 0)
                      : launch(tf32x3_gemm_kernel<true, 64, false>, bhi_blocked ? 1 : 0));
  } else {
    PGB_TRY(bn == 256 ? launch(tf32x3_gemm_kernel<false, 256, false>, 0)
                      : launch(tf32x3_gemm_kernel<false, 64, false>, 0));
  }
  note_launch(PATH_TCGEN05);
  PGB_CUDA(cudaGetLastError());
  return PGB200_OK;
}

// Test hook (host only): the (tile row, tile column) sequence the fp32 kernels
// walk for an M x N output with the given tile shape, as TileCursor yields it.
// Returns the number of tiles, or -1 when `cap` pairs do not hold them.
int64_t enumerate_tiles_for_test(int64_t M, int64_t N, int bm, int bn, int lower, int64_t row0,
                                 int64_t *tm_out, int64_t *tn_out, int64_t cap) {
  Tiles t = {};
  t.tiles_m = (M + bm - 1) / bm;
  t.tiles_n = (N + bn - 1) / bn;
  t.bm = bm;
  t.bn = bn;
  t.lower = lower;
  t.row0 = row0;
  t.splits = 1;
  t.total = count_tiles(t);
  if (t.total > cap) return -1;
  TileCursor cur;
  for (int64_t i = 0; i < t.total; i++) cur.seek(t, i, &tm_out[i], &tn_out[i]);
  return t.total;
}

}  // namespace pgb200
