// Prefill attention on the fifth-generation tensor cores (tcgen05.mma), for bfloat16, head size 128
// and groups of up to 32 query heads per kv head.  Same contract and formulas as
// attention_mma.cu (pygguf_engine/kv_cache.py:833, 2189-2192 masks; 756 head mapping; 836-861 online
// softmax); other shapes keep using that file.
//
// A block owns up to 128 rows of one (sequence, kv head), a row being a (query token, head of the
// group) pair: 128 / group whole tokens (a group of 5 gives 125 rows; the rest of the MMA's 128 rows is
// zero and is never stored).  It walks the sequence's 64-key pages.  Roles:
//   warp 5    TMA producer: Q once (a 3-D box [tokens][group heads][64 features] per feature half),
//             then K pages into a ring of two (a K page is spent as soon as S is there) and V pages
//             into a ring of three (needed until P.V), so that a page's copy starts two pages ahead.  The
//             first page's K has a barrier of its own; after it, a page's V and the next page's K are
//             copied onto one barrier;
//   warp 4    MMA issuer: S = Q.K^T (128 x 64, eight k-steps of 16) into one of two S accumulators in
//             tensor memory, and O += P.V (128 x 128, four k-steps of 16 keys) with P as the A operand
//             from tensor memory and V as an MN-major operand from shared memory, so the page that TMA
//             wrote as [keys][features] needs no transpose.  Its loop is what a block's pace hangs on, and
//             it is one thread: per page it waits three times and commits twice (see the barriers' list);
//   warps 0-3 softmax: thread r owns row r.  It reads its S row from TMEM (tcgen05.ld), scales and
//             masks (pages below the diagonal need no mask), keeps the running maximum and sum in
//             registers, writes P as bfloat16 pairs back over the S columns it has read (tcgen05.st: P
//             never touches shared memory), and rescales its O row in TMEM (tcgen05.ld / tcgen05.st)
//             only when the maximum has grown by more than 2^8 since the last rescale (the reference of
//             the exponentials is then moved; until then P simply carries the larger factor, which
//             float32 sums and bfloat16 products hold without loss).
// S of page j + 2 overwrites the columns of P of page j: warp 4 issues it only after P.V of page j
// has completed.
// S of the next page is computed while the softmax of the current one runs.  All waits are bounded.
//
// Blocks are persistent: the grid is two blocks per SM (or fewer, if there is less work), and each block
// takes several work items, an item being the 128 rows of one (row tile, sequence, kv head).  Items are
// ranked with the late row tiles first (under the causal mask they see the most pages).  With a work
// counter (two ints in global memory, zero before the launch and zero again after it) a block takes the
// next rank whenever it is free, so the light items at the end even out what the heavy ones left uneven;
// without one, ranks are dealt out in a serpentine (block c takes ranks c, 2G-1-c, 2G+c, ... of a grid
// of G blocks).  One 2,048-token prompt with 8 kv heads is 512 items of 1 to 32 pages: a launch of 512
// blocks in 1.73 waves on 296 slots left the SMs half empty for the second wave.  Which block computes an
// item changes nothing in its result (the counter only hands out ranks; no sum depends on it).  The
// producer warp fetches the rank and hands it to the other warps through a two-slot ring in shared memory.
// Barrier phases, the K/V rings and tensor memory carry over from item to item: every role counts items
// and pages the same way.
#include "api.h"
#include "common.cuh"
#include "tma.cuh"

namespace pe {
namespace fau {

constexpr int HD = 128;        // head size
constexpr int BM = 128;        // rows per block
constexpr int BN = 64;         // keys per page
constexpr int kQBytes = BM * HD * 2;          // 32 KB: two 64-feature halves of [128 rows][128 B]
constexpr int kPageBytes = BN * HD * 2;        // 16 KB: a K or V page, two halves of [64][128 B]
constexpr int kKStages = 2, kVStages = 3;     // K is spent once S is there, V only after P.V: V needs the deeper ring
constexpr int kTmemCols = 256;                // S0 [0,64) S1 [64,128) O [128,256)
constexpr float kRescaleThreshold = 8.0f;     // in log2 units

struct Args {
  __nv_bfloat16* out; long long out_ld;
  int n_heads, n_kv_heads, group;
  float scale_log2;
  int window;
  const int* seq_qstart; const int* seq_past; const int* seq_slot;
  const int* page_table; int table_stride; int num_pages;
  int* status;
  int tiles, n_seqs;      // row tiles of the step's longest sequence; sequences
  int* work_counter;      // [0] next rank, [1] blocks that are through; both zero between launches.  May be null.
};

// One work item: the rows [row0, row0 + rows_blk) of sequence b's (token, head) rows for kv head kvh.
struct Item {
  int b, kvh, row0, n_rows, q0, past, slot, tok0, k_begin, n_tiles;
};
// Rank -> item (late row tiles first, then sequences, then kv heads); false if the sequence has no such rows.
__device__ __forceinline__ bool item_at(const Args& a, int rank, int rows_blk, Item& w) {
  w.kvh = rank % a.n_kv_heads;
  const int r2 = rank / a.n_kv_heads;
  w.b = r2 % a.n_seqs;
  const int tile = a.tiles - 1 - r2 / a.n_seqs;
  w.q0 = a.seq_qstart[w.b];
  const int q_len = a.seq_qstart[w.b + 1] - w.q0;
  w.past = a.seq_past[w.b];
  w.n_rows = q_len * a.group;
  w.row0 = tile * rows_blk;
  if (w.row0 >= w.n_rows) return false;
  w.slot = a.seq_slot[w.b];
  w.tok0 = w.row0 / a.group;
  const int last_row = min(w.n_rows, w.row0 + rows_blk) - 1;
  const int first_pos = w.past + w.tok0, last_pos = w.past + last_row / a.group;
  w.k_begin = 0;
  if (a.window > 0) w.k_begin = max(0, first_pos - a.window + 1) / BN * BN;
  w.n_tiles = (last_pos + 1 - w.k_begin + BN - 1) / BN;
  return true;
}
// Every block calls this once, when it takes no more ranks: the last of the G blocks through leaves the work
// counter as it found it, zero (also on the error paths, or the next launch would find no work).
__device__ __forceinline__ void leave_work_counter(int* counter, int G) {
  if (counter == nullptr) return;
  __threadfence();
  if (atomicAdd(counter + 1, 1) == G - 1) {
    counter[0] = 0;
    counter[1] = 0;
    __threadfence();
  }
}
// The rank that block c of G takes in pass p (serpentine), or -1 when the passes are over.
__device__ __forceinline__ int rank_of(int pass, int c, int G, int total) {
  if (pass * G >= total) return -1;
  const int rank = (pass & 1) ? (pass + 1) * G - 1 - c : pass * G + c;
  return rank < total ? rank : total;      // total: nothing for this block in this pass
}

// ---- tcgen05 wrappers (see gemm_umma.cu for the descriptor layouts) ------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t* holder, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(tma::smem_addr(holder)), "r"(cols));
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::);
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(taddr), "r"(cols));
}
__device__ __forceinline__ void fence_before_sync() { asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void fence_after_sync() { asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(tma::smem_addr(bar)) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,"
      "%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];\n"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr));
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,"
      "%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};\n" ::"r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
      "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]),
      "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]),
      "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory"); }
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory"); }

// kind::f16 instruction descriptor: float32 D, bfloat16 A and B, A K-major; b_mn: B is MN-major (bit 16).
__host__ __device__ constexpr uint32_t instr_desc(int m, int n, bool b_mn) {
  return (1u << 4) | (1u << 7) | (1u << 10) | (b_mn ? (1u << 16) : 0u) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

// The MMA-issuing thread is one thread that issues one instruction after the other, and its loop sets a block's
// pace: a product's k-step or a commit costs it some 70 cycles, a wait well over a hundred even on a barrier that is
// long complete.  Whatever it does between those counts as well: the 64-bit operand descriptors' constant upper
// word (1,024 bytes between 8-row groups, descriptor version, 128-byte swizzle) is set once, the lower word
// (start address in 16-byte units; for an MN-major operand also the distance between its two 64-column halves)
// is advanced by adding constants, and the k-steps of a product are issued from one block of instructions.
constexpr uint32_t kDescHi = (1024u >> 4) | (1u << 14) | (2u << 29);
// K-major operand, 128-byte swizzle: rows of 128 bytes, 8-row groups 1,024 bytes apart.
__device__ __forceinline__ uint32_t desc_lo_k_major(uint32_t saddr) { return ((saddr >> 4) & 0x3FFF) | (1u << 16); }
// MN-major operand, 128-byte swizzle: 64 elements of the N dimension are contiguous (128 bytes); the next 64 lie
// `lbo` bytes further; along K, rows are 128 bytes apart in groups of 8 (1,024 bytes).
__device__ __forceinline__ uint32_t desc_lo_mn_major(uint32_t saddr, uint32_t lbo_bytes) {
  return ((saddr >> 4) & 0x3FFF) | (((lbo_bytes >> 4) & 0x3FFF) << 16);
}

// S = Q.K^T of one page: eight k-steps of 16 features.  Both operands are two 64-feature halves of [rows][128 B]:
// a k-step moves 32 bytes (2 units) inside a half, the second half lies rows * 128 bytes further (A: 128 rows,
// 1,024 units; B: 64 keys, 512 units).
#define PE_QK_STEP(A, B)                                                                       \
  "add.u32 al, %1, " #A ";\n"                                                                  \
  "add.u32 bl, %2, " #B ";\n"                                                                  \
  "mov.b64 da, {al, %3};\n"                                                                    \
  "mov.b64 db, {bl, %3};\n"                                                                    \
  "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %4, pt;\n"
__device__ __forceinline__ void umma_qk_page(uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo, uint32_t idesc) {
  asm volatile(
      "{\n"
      ".reg .pred pf, pt;\n"
      ".reg .b64 da, db;\n"
      ".reg .b32 al, bl;\n"
      "setp.ne.b32 pf, %4, %4;\n"
      "setp.eq.b32 pt, %4, %4;\n"
      "mov.b64 da, {%1, %3};\n"
      "mov.b64 db, {%2, %3};\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %4, pf;\n"
      PE_QK_STEP(2, 2) PE_QK_STEP(4, 4) PE_QK_STEP(6, 6)
      PE_QK_STEP(1024, 512) PE_QK_STEP(1026, 514) PE_QK_STEP(1028, 516) PE_QK_STEP(1030, 518)
      "}\n" ::"r"(d_tmem), "r"(a_lo), "r"(b_lo), "r"(kDescHi), "r"(idesc) : "memory");
}
#undef PE_QK_STEP
// O (+)= P.V of one page: four k-steps of 16 keys.  P comes from tensor memory (8 columns of bfloat16 pairs a
// step), V is MN-major: 16 keys are 16 rows of 128 bytes (128 units).  `accumulate` == 0: the first step starts O.
#define PE_PV_STEP(T, B)                                                                       \
  "add.u32 ta, %1, " #T ";\n"                                                                  \
  "add.u32 bl, %2, " #B ";\n"                                                                  \
  "mov.b64 db, {bl, %3};\n"                                                                    \
  "tcgen05.mma.cta_group::1.kind::f16 [%0], [ta], db, %4, pt;\n"
__device__ __forceinline__ void umma_pv_page(uint32_t d_tmem, uint32_t p_tmem, uint32_t v_lo, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p0, pt;\n"
      ".reg .b64 db;\n"
      ".reg .b32 ta, bl;\n"
      "setp.ne.b32 p0, %5, 0;\n"
      "setp.eq.b32 pt, %4, %4;\n"
      "mov.b64 db, {%2, %3};\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], db, %4, p0;\n"
      PE_PV_STEP(8, 128) PE_PV_STEP(16, 256) PE_PV_STEP(24, 384)
      "}\n" ::"r"(d_tmem), "r"(p_tmem), "r"(v_lo), "r"(kDescHi), "r"(idesc), "r"(accumulate) : "memory");
}
#undef PE_PV_STEP
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
  return y;
}
// Blackwell's two-wide float32 arithmetic and three-input maximum: the softmax threads are bound by the number
// of instructions they issue, not by any one pipe.
__device__ __forceinline__ float max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;\n" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}
__device__ __forceinline__ uint64_t pack_f32x2(float lo, float hi) {
  uint64_t v;
  asm("mov.b64 %0, {%1, %2};\n" : "=l"(v) : "f"(lo), "f"(hi));
  return v;
}
__device__ __forceinline__ void unpack_f32x2(uint64_t v, float& lo, float& hi) {
  asm("mov.b64 {%0, %1}, %2;\n" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ uint64_t fma_f32x2(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;\n" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}
__device__ __forceinline__ uint64_t add_f32x2(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("add.rn.f32x2 %0, %1, %2;\n" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ void load_3d(void* dst, const CUtensorMap* map, int x, int y, int z, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];\n"
      ::"r"(tma::smem_addr(dst)), "l"(map), "r"(x), "r"(y), "r"(z), "r"(tma::smem_addr(bar)) : "memory");
}

// grid: G persistent blocks (see the file's head); block: 192 threads.
__global__ void __launch_bounds__(192, 2)
prefill_umma_kernel(Args a, const __grid_constant__ CUtensorMap qmap, const __grid_constant__ CUtensorMap kmap,
                    const __grid_constant__ CUtensorMap vmap) {
  // All shared memory is dynamic and starts on a 1,024-byte boundary (there are no static shared
  // variables in front of it), so that two blocks fit on an SM: tiles first, barriers behind them.
  extern __shared__ __align__(1024) char smem[];
  char* q_s = smem;                       // [2 halves][128 rows][128 B]
  char* k_s = q_s + kQBytes;              // kKStages K pages
  char* v_s = k_s + kKStages * kPageBytes;   // kVStages V pages
  uint64_t* bars = reinterpret_cast<uint64_t*>(v_s + kVStages * kPageBytes);
  uint64_t& q_full = bars[0];
  // The MMA thread's commits are few on purpose: that thread issues one instruction after the other, a commit costs
  // it about as much as a product's k-step, and its loop sets a block's pace.  So a barrier serves every purpose it
  // can: S of a page being there also says that the page's K stage is spent (a K stage and an S buffer have the
  // same index), and a V stage being spent also says that the page's P.V product is done.
  uint64_t& k0_full = bars[1];    // one phase per item: K of its first page is there
  uint64_t* kv_full = bars + 5;   // [3], by V stage: V of a page and K of the page after it (copied together, so that
                                  //      the MMA thread waits once a page for both) are there
  uint64_t* v_empty = bars + 8;   // [3]: the page's P.V product is done: the stage may be filled again, O may be
                                  //      rescaled, the S after next may overwrite the page's P
  uint64_t* s_full = bars + 11;   // [2]: S of a page is in the buffer, and the page's K stage may be filled again
  uint64_t* p_ready = bars + 13;  // [2]: one per S buffer, the softmax may be a page ahead of the P.V products
  uint64_t& o_done = bars[16];    // one phase per item: its last P.V product is done.  (A barrier of its own: the
                                  // softmax does not follow the pages' products phase by phase, and a parity wait
                                  // that is two phases ahead of its barrier passes at once.)
  uint64_t& q_empty = bars[17];   // one phase per item: its last S product has read Q
  uint64_t& o_free = bars[18];    // one phase per item: the softmax threads have read O out
  uint64_t* w_full = bars + 19;   // [2]: a rank has been put into the slot
  uint64_t* w_empty = bars + 21;  // [2]: the MMA thread and the 128 softmax threads have read it
  uint32_t& tmem_holder = *reinterpret_cast<uint32_t*>(bars + 23);
  volatile int& failed = *reinterpret_cast<volatile int*>(bars + 24);
  volatile int* work_slot = reinterpret_cast<volatile int*>(bars + 25);   // [2] ranks; -1: no more work
  if ((tma::smem_addr(smem) & 1023u) != 0) {   // the swizzled tiles need this alignment
    if (threadIdx.x == 0) {
      report(a.status, kStatusWaitTimedOut, 29, (int)(tma::smem_addr(smem) & 1023u), 0);
      leave_work_counter(a.work_counter, (int)gridDim.x);
    }
    return;
  }
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int group = a.group;
  const int rows_blk = (BM / group) * group;                  // whole tokens only
  const int G = (int)gridDim.x, me = (int)blockIdx.x;
  const int total = a.tiles * a.n_seqs * a.n_kv_heads;

  if (tid == 0) {
    tma::mbar_init(&q_full, 1);
    tma::mbar_init(&k0_full, 1);
    for (int s = 0; s < 2; ++s) {
      tma::mbar_init(&s_full[s], 1);
      tma::mbar_init(&p_ready[s], 128);
    }
    for (int s = 0; s < kVStages; ++s) {
      tma::mbar_init(&kv_full[s], 1);
      tma::mbar_init(&v_empty[s], 1);
    }
    tma::mbar_init(&o_done, 1);
    tma::mbar_init(&q_empty, 1);
    tma::mbar_init(&o_free, 128);
    for (int s = 0; s < 2; ++s) {
      tma::mbar_init(&w_full[s], 1);
      tma::mbar_init(&w_empty[s], 129);
    }
    failed = 0;
    tma::fence_barrier_init();
  }
  // the Q rows beyond the block's whole tokens are no copy's target: zero them (both feature halves)
  // so that the MMA's rows there stay finite; they are never stored
  for (int i = tid; i < (BM - rows_blk) * 2 * 8; i += blockDim.x) {
    const int rr = rows_blk + i / 16, half = (i / 8) & 1, chunk = i & 7;
    *reinterpret_cast<uint4*>(q_s + half * (kQBytes / 2) + rr * 128 + chunk * 16) = make_uint4(0, 0, 0, 0);
  }
  tma::fence_proxy_async();
  if (warp == 4) tmem_alloc(&tmem_holder, kTmemCols);
  fence_before_sync();
  // Barriers, the zeroed Q rows and tensor memory touch nothing that another kernel of the step writes: all of
  // that is done while the kernel before may still be draining; only now wait for it (its output is q, K, V).
  pdl_wait_block();
  pdl_launch_dependents();
  fence_after_sync();
  const uint32_t tmem_base = tmem_holder;
  const uint32_t tmem_o = tmem_base + 128;

  // Every role walks the same items in the same order and counts alike: `it` items done, `n` pages done.
  uint32_t it = 0, n = 0;
  if (warp == 5) {
    // ---- TMA producer ----
    if (lane == 0) {
      for (uint32_t f = 0;; ++f) {
        // the next rank: from the counter, or by the serpentine; into the ring for the other warps
        int rank = -1;
        if (!failed) {
          if (a.work_counter != nullptr) {
            rank = atomicAdd(a.work_counter, 1);
            if (rank >= total) rank = -1;
          } else {
            rank = rank_of((int)f, me, G, total);
          }
          if (f >= 2 && !tma::mbar_wait(&w_empty[f & 1], ((f >> 1) & 1) ^ 1)) {
            report(a.status, kStatusWaitTimedOut, 26, me, (int)f);
            failed = 1;
            rank = -1;
          }
        }
        work_slot[f & 1] = rank;
        tma::mbar_arrive(&w_full[f & 1]);
        if (rank < 0) break;
        Item w;
        if (rank >= total || !item_at(a, rank, rows_blk, w)) continue;
        // Q of the item before must have been read by its last S product
        if (!tma::mbar_wait(&q_empty, (it & 1) ^ 1)) {
          report(a.status, kStatusWaitTimedOut, 25, me, (int)it);
          failed = 1;
          continue;              // the loop's head then tells the other warps that nothing follows
        }
        tma::mbar_expect_tx(&q_full, (uint32_t)(rows_blk * HD * 2));
        load_3d(q_s, &qmap, 0, w.kvh * group, w.q0 + w.tok0, &q_full);
        load_3d(q_s + kQBytes / 2, &qmap, 64, w.kvh * group, w.q0 + w.tok0, &q_full);
        // Row of the page table's page for the item's page j in the K and V tensors' 2-D views.
        auto page_row = [&](int j) -> int {
          const int k0 = w.k_begin + j * BN;
          const int logical = k0 / BN;
          int page = -1;
          if (logical < a.table_stride) page = a.page_table[(size_t)w.slot * a.table_stride + logical];
          if (page < 0 || page >= a.num_pages) {
            report(a.status, kStatusPageOutOfRange, w.slot, page, k0);
            page = 0;
          }
          return (page * a.n_kv_heads + w.kvh) * BN;
        };
        // K of page g goes into K stage g mod 2, which is free once S of page g - 2 is there (the S buffer of that
        // index has the stage's number)
        auto k_stage_free = [&](uint32_t g) -> bool {
          return tma::mbar_wait(&s_full[g % kKStages], ((g / kKStages) & 1) ^ 1);
        };
        auto load_k = [&](uint32_t g, int y, uint64_t* bar) {
          char* kd = k_s + (g % kKStages) * kPageBytes;
          tma::load_2d(kd, &kmap, 0, y, bar);
          tma::load_2d(kd + BN * 128, &kmap, 64, y, bar);
        };
        int y = page_row(0);
        // the first page's K alone; every later K page travels with the V page before it
        if (!k_stage_free(n)) {
          report(a.status, kStatusWaitTimedOut, 20, me, 0);
          failed = 1;
          continue;
        }
        tma::mbar_expect_tx(&k0_full, kPageBytes);
        load_k(n, y, &k0_full);
        for (int j = 0; j < w.n_tiles && !failed; ++j) {
          const uint32_t g = n + j;
          const int vs = g % kVStages;
          const bool more = j + 1 < w.n_tiles;
          const int y_next = more ? page_row(j + 1) : 0;
          if (!tma::mbar_wait(&v_empty[vs], ((g / kVStages) & 1) ^ 1) || (more && !k_stage_free(g + 1))) {
            report(a.status, kStatusWaitTimedOut, 24, me, j);
            failed = 1;
            break;
          }
          char* vd = v_s + vs * kPageBytes;
          tma::mbar_expect_tx(&kv_full[vs], more ? 2 * kPageBytes : kPageBytes);
          tma::load_2d(vd, &vmap, 0, y, &kv_full[vs]);
          tma::load_2d(vd + BN * 128, &vmap, 64, y, &kv_full[vs]);
          if (more) load_k(g + 1, y_next, &kv_full[vs]);
          y = y_next;
        }
        n += w.n_tiles;
        ++it;
      }
    }
  } else if (warp == 4) {
    // ---- MMA issuer ----
    if (lane == 0) {
      const uint32_t idesc_qk = instr_desc(BM, BN, false);
      const uint32_t idesc_pv = instr_desc(BM, HD, true);
      const uint32_t q_lo = desc_lo_k_major(tma::smem_addr(q_s));
      const uint32_t k_lo0 = desc_lo_k_major(tma::smem_addr(k_s));               // stage s: + s * (16 KB / 16)
      const uint32_t v_lo0 = desc_lo_mn_major(tma::smem_addr(v_s), BN * 128);
      bool ok = true;
      for (uint32_t f = 0; ok && !failed; ++f) {
        if (!tma::mbar_wait(&w_full[f & 1], (f >> 1) & 1)) { ok = false; break; }
        const int rank = work_slot[f & 1];
        tma::mbar_arrive(&w_empty[f & 1]);
        if (rank < 0) break;
        Item w;
        if (rank >= total || !item_at(a, rank, rows_blk, w)) continue;
        const int n_tiles = w.n_tiles;
        // S of the item's page j; its K page is there (the caller has waited for the barrier that counts it)
        auto issue_qk = [&](int j) {
          const uint32_t g = n + j;
          const int st = g & 1, ks = g % kKStages;
          fence_after_sync();
          umma_qk_page(tmem_base + st * BN, q_lo, k_lo0 + ((uint32_t)ks << 10), idesc_qk);
          umma_commit(&s_full[st]);     // S is there, and the K stage is spent
          if (j == n_tiles - 1) umma_commit(&q_empty);   // ... and so is Q, after the item's last S product
        };
        ok = tma::mbar_wait(&q_full, it & 1) && tma::mbar_wait(&k0_full, it & 1);
        if (ok) issue_qk(0);
        for (int j = 0; ok && j < n_tiles; ++j) {
          const uint32_t g = n + j;
          // S of page j + 1 goes where P of page j - 1 lies: that P.V product must have read it.  (Products
          // of one thread run in issue order on today's hardware; the wait makes the order explicit and
          // costs nothing, the softmax of page j is still running.)  Across items nothing is pending: an
          // item ends with all its products complete.
          if (j >= 1 && j + 1 < n_tiles && !tma::mbar_wait(&v_empty[(g - 1) % kVStages], ((g - 1) / kVStages) & 1)) { ok = false; break; }
          const int st = g & 1, vs = g % kVStages;
          // V of this page and K of the next arrive together
          if (!tma::mbar_wait(&kv_full[vs], (g / kVStages) & 1)) { ok = false; break; }
          if (j + 1 < n_tiles) issue_qk(j + 1);             // S of the next page while this one's softmax runs
          if (!tma::mbar_wait(&p_ready[st], (g >> 1) & 1)) { ok = false; break; }
          // the first product of an item starts O anew: the item before must have been read out of it
          if (j == 0 && !tma::mbar_wait(&o_free, (it & 1) ^ 1)) { ok = false; break; }
          fence_after_sync();
          // P lies where S of this page was (bfloat16 pairs, 32 columns)
          umma_pv_page(tmem_o, tmem_base + st * BN, v_lo0 + ((uint32_t)vs << 10), idesc_pv, j > 0 ? 1u : 0u);
          umma_commit(&v_empty[vs]);    // the V page is spent, and whoever waits for this product may go on
        }
        if (ok) {
          umma_commit(&o_done);
          // the item ends with every product complete: the next item's S products overwrite the P columns
          ok = tma::mbar_wait(&o_done, it & 1);
        }
        n += n_tiles;
        ++it;
      }
      if (!ok) {
        report(a.status, kStatusWaitTimedOut, 21, me, (int)it);
        failed = 1;
      }
    }
  } else {
    // ---- softmax: thread r owns row r ----
    const int r = tid;                               // 0..127; warp w reads TMEM lanes 32w..32w+31
    const uint32_t lane_off = (uint32_t)(warp * 32) << 16;
    bool ok = true;
    for (uint32_t f = 0; ok && !failed; ++f) {
      if (!tma::mbar_wait(&w_full[f & 1], (f >> 1) & 1)) {
        if (lane == 0) report(a.status, kStatusWaitTimedOut, 27, me, (int)f);
        failed = 1;
        break;
      }
      const int rank = work_slot[f & 1];
      tma::mbar_arrive(&w_empty[f & 1]);
      if (rank < 0) break;
      Item w;
      if (rank >= total || !item_at(a, rank, rows_blk, w)) continue;
      const int row0 = w.row0, n_rows = w.n_rows, past = w.past, n_tiles = w.n_tiles;
      const int row = row0 + r;
      const bool live = r < rows_blk && row < n_rows;
      const int qpos = past + row / group;
      float m_ref = -INFINITY, l = 0.f;
      for (int j = 0; j < n_tiles; ++j) {
        const uint32_t g = n + j;
        const int st = g & 1;
        const int k0 = w.k_begin + j * BN;
        if (failed || !tma::mbar_wait(&s_full[st], (g >> 1) & 1)) { ok = false; break; }
        fence_after_sync();
        uint32_t sv[2][32];
        tmem_ld32(tmem_base + st * BN + lane_off, sv[0]);
        tmem_ld32(tmem_base + st * BN + 32 + lane_off, sv[1]);
        tmem_ld_wait();
        // A page that every row of this block sees whole (below the diagonal, inside the window) needs
        // no mask: the scores stay raw and the scale is folded into the exponent's multiply-add.
        const bool whole = a.scale_log2 > 0.f && (row0 + rows_blk <= n_rows) && (k0 + BN - 1 <= past + row0 / group) &&
                           (a.window <= 0 || k0 > past + (row0 + rows_blk - 1) / group - a.window);
        float mx = -INFINITY;
        if (whole) {
          // four independent chains: a thread has few other warps to hide a 64-long dependent chain behind
          float m4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
          for (int h = 0; h < 2; ++h)
#pragma unroll
            for (int c = 0; c < 16; ++c)
              m4[c & 3] = max3(m4[c & 3], __uint_as_float(sv[h][2 * c]), __uint_as_float(sv[h][2 * c + 1]));
          mx = fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3])) * a.scale_log2;   // the scale is positive
        } else {
#pragma unroll
          for (int h = 0; h < 2; ++h)
#pragma unroll
            for (int c = 0; c < 32; ++c) {
              const int kpos = k0 + h * 32 + c;
              bool vis = live && kpos <= qpos;
              if (a.window > 0) vis = vis && (kpos > qpos - a.window);
              const float v = vis ? __uint_as_float(sv[h][c]) * a.scale_log2 : -INFINITY;
              sv[h][c] = __float_as_uint(v);
              mx = fmaxf(mx, v);
            }
        }
        // move the reference of the exponentials only when the maximum has grown a lot
        const bool grow = mx > m_ref + kRescaleThreshold;
        if (__any_sync(0xffffffffu, grow && j > 0 && m_ref != -INFINITY)) {
          // O is rescaled in place: the previous P.V must be done with it first
          if (!tma::mbar_wait(&v_empty[(g - 1) % kVStages], ((g - 1) / kVStages) & 1)) { ok = false; break; }
          fence_after_sync();
          const float f = (grow && m_ref != -INFINITY) ? fast_exp2(m_ref - mx) : 1.0f;
#pragma unroll 1
          for (int c = 0; c < HD; c += 32) {
            uint32_t ov[32];
            tmem_ld32(tmem_o + c + lane_off, ov);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) ov[i] = __float_as_uint(__uint_as_float(ov[i]) * f);
            tmem_st32(tmem_o + c + lane_off, ov);
          }
          tmem_st_wait();
          l *= f;
        }
        if (grow) m_ref = mx;
        const float base = (m_ref == -INFINITY) ? 0.f : m_ref;
        uint64_t sum4[4] = {0ull, 0ull, 0ull, 0ull};   // four chains of two-wide sums; added up in a fixed order below
        // P = exp2(score - reference) as bfloat16 pairs, back into tensor memory where S of this page was
        // (this thread has read all of its S row): the P.V product takes its A operand from there.  Scale and
        // reference go in as one two-wide multiply-add per pair of scores (masked scores are scaled already).
        uint32_t pw[32];
        const float sc = whole ? a.scale_log2 : 1.0f, nb = -base;
        const uint64_t sc2 = pack_f32x2(sc, sc), nb2 = pack_f32x2(nb, nb);
#pragma unroll
        for (int h = 0; h < 2; ++h)
#pragma unroll
          for (int c = 0; c < 16; ++c) {
            float x0, x1;
            unpack_f32x2(fma_f32x2(pack_f32x2(__uint_as_float(sv[h][2 * c]), __uint_as_float(sv[h][2 * c + 1])), sc2, nb2), x0, x1);
            const float p0 = fast_exp2(x0), p1 = fast_exp2(x1);
            sum4[c & 3] = add_f32x2(sum4[c & 3], pack_f32x2(p0, p1));
            pw[h * 16 + c] = pack2(p0, p1);
          }
        tmem_st32(tmem_base + st * BN + lane_off, pw);
        tmem_st_wait();
        {
          float s0, s1, s2, s3, s4, s5, s6, s7;
          unpack_f32x2(sum4[0], s0, s1); unpack_f32x2(sum4[1], s2, s3);
          unpack_f32x2(sum4[2], s4, s5); unpack_f32x2(sum4[3], s6, s7);
          l += ((s0 + s1) + (s2 + s3)) + ((s4 + s5) + (s6 + s7));
        }
        fence_before_sync();
        tma::mbar_arrive(&p_ready[st]);
      }
      if (ok && tma::mbar_wait(&o_done, it & 1)) {
        fence_after_sync();
        const float inv = 1.f / fmaxf(l, 1e-20f);
        const int tok = row / group, head = w.kvh * group + row % group;
        __nv_bfloat16* dst = a.out + (size_t)(w.q0 + tok) * a.out_ld + (size_t)head * HD;
#pragma unroll 1
        for (int c = 0; c < HD; c += 32) {
          uint32_t ov[32];
          tmem_ld32(tmem_o + c + lane_off, ov);
          tmem_ld_wait();
          if (live) {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              uint4 o4;
              o4.x = pack2(__uint_as_float(ov[8 * i]) * inv, __uint_as_float(ov[8 * i + 1]) * inv);
              o4.y = pack2(__uint_as_float(ov[8 * i + 2]) * inv, __uint_as_float(ov[8 * i + 3]) * inv);
              o4.z = pack2(__uint_as_float(ov[8 * i + 4]) * inv, __uint_as_float(ov[8 * i + 5]) * inv);
              o4.w = pack2(__uint_as_float(ov[8 * i + 6]) * inv, __uint_as_float(ov[8 * i + 7]) * inv);
              *reinterpret_cast<uint4*>(dst + c + 8 * i) = o4;
            }
          }
        }
        // O has been read out: the next item's first P.V product may start it anew
        fence_before_sync();
        tma::mbar_arrive(&o_free);
      } else {
        if (lane == 0 && !failed) report(a.status, kStatusWaitTimedOut, 22, me, (int)it);
        failed = 1;
        ok = false;
      }
      n += n_tiles;
      ++it;
    }
  }
  fence_before_sync();
  __syncthreads();
  if (warp == 4) {
    fence_after_sync();
    tmem_dealloc(tmem_base, kTmemCols);
  }
  if (tid == 0) leave_work_counter(a.work_counter, G);
}

}  // namespace fau
}  // namespace pe

extern "C" int pe_attention_umma_supported(int head_dim, int n_heads, int n_kv_heads) {
  if (head_dim != 128 || n_kv_heads <= 0 || n_heads % n_kv_heads) return 0;
  const int g = n_heads / n_kv_heads;
  return (g >= 1 && g <= 32) ? 1 : 0;
}

// Prefill form only (decode keeps attention_mma.cu).  q: rows of the fused q|k|v buffer, [n_tokens, q_ld].
// n_sms: the device's SM count (sizes the persistent grid).  work_counter: two ints, zero before the call (the
// kernel leaves them zero), not shared with a call that may run at the same time; null: a fixed schedule.
extern "C" int pe_attention_umma_prefill(const void* q, long long q_ld, long long n_tokens, void* out, long long out_ld,
                                         int n_seqs, int max_q, int n_heads, int n_kv_heads, int head_dim, float scale,
                                         int window, const int* seq_qstart, const int* seq_past, const int* seq_slot,
                                         const int* page_table, int table_stride, int num_pages, const void* k_pages,
                                         const void* v_pages, int n_sms, int* work_counter, int* status, cudaStream_t stream) {
  using namespace pe::fau;
  if (n_seqs <= 0) return PE_OK;
  if (!pe_attention_umma_supported(head_dim, n_heads, n_kv_heads)) return PE_ERR_UNSUPPORTED_SIZE;
  if (((uintptr_t)q % 16) || (q_ld * 2) % 16 || ((uintptr_t)out % 16) || (out_ld * 2) % 16) return PE_ERR_BAD_ARGUMENT;
  Args a;
  a.out = (__nv_bfloat16*)out; a.out_ld = out_ld; a.n_heads = n_heads; a.n_kv_heads = n_kv_heads;
  a.group = n_heads / n_kv_heads; a.scale_log2 = scale * 1.4426950408889634f; a.window = window;
  a.seq_qstart = seq_qstart; a.seq_past = seq_past; a.seq_slot = seq_slot;
  a.page_table = page_table; a.table_stride = table_stride; a.num_pages = num_pages; a.status = status;
  pe::tma::EncodeTiledFn fn = pe::tma::encode_fn();
  if (fn == nullptr) return -5;
  CUtensorMap qmap, kmap, vmap;
  {
    cuuint64_t dims[3] = {(cuuint64_t)HD, (cuuint64_t)n_heads, (cuuint64_t)n_tokens};
    cuuint64_t strides[2] = {(cuuint64_t)HD * 2, (cuuint64_t)q_ld * 2};
    cuuint32_t box[3] = {64, (cuuint32_t)a.group, (cuuint32_t)(BM / a.group)};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = fn(&qmap, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(q), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return PE_ERR_BAD_ARGUMENT;
  }
  const uint64_t rows = (uint64_t)num_pages * n_kv_heads * BN;
  int me = pe::tma::make_map_2d_bf16(&kmap, k_pages, HD, rows, HD, 64, BN);
  if (me == 0) me = pe::tma::make_map_2d_bf16(&vmap, v_pages, HD, rows, HD, 64, BN);
  if (me != 0) return me < 0 ? me : PE_ERR_BAD_ARGUMENT;
  const size_t smem = kQBytes + (kKStages + kVStages) * kPageBytes + 256;   // tiles, then barriers and the two-slot ring
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t ce = cudaFuncSetAttribute(prefill_umma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (ce != cudaSuccess) return (int)ce;
    attr_set = true;
  }
  const int rows_blk = (BM / a.group) * a.group;
  const long long tiles = ((long long)max_q * a.group + rows_blk - 1) / rows_blk;
  const long long total = tiles * n_kv_heads * n_seqs;
  if (total <= 0 || total > (1ll << 30)) return PE_ERR_UNSUPPORTED_SIZE;
  a.tiles = (int)tiles; a.n_seqs = n_seqs; a.work_counter = work_counter;
  // two blocks fit on an SM (shared memory, tensor memory columns); no more blocks than items
  const long long slots = 2ll * (n_sms > 0 ? n_sms : pe::kSMs);
  dim3 grid((unsigned)(total < slots ? total : slots));
  pe::launch(prefill_umma_kernel, grid, 192, smem, stream, a, qmap, kmap, vmap);
  PE_LAUNCH_CHECK();
  return PE_OK;
}
