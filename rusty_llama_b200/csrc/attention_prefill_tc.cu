// Causal flash attention for prompts on the 5th-generation tensor cores, head sizes 64 and 128, bfloat16,
// reading keys and values from the paged cache.  Same contract as `flash_prefill` (ragged batch,
// positions from seq_pos0, optional window); the reference's counterpart is its scalar
// `attention_kernel` (src/backend/cuda.rs:157-232).
//
// A block owns 128 query rows of one head of one sequence and walks over key tiles of 64
// positions (one cache page):
//   warp 4 (one lane)  TMA: the Q tile once, then K and V tiles (64 x 64 boxes straight from their
//                      page, 128-byte swizzled) into two-stage rings;
//   warp 5 (one lane)  tcgen05.mma: S = Q K^T (128 x 64, k = head size) into one of two S buffers
//                      in tensor memory, always one tile ahead; then O += P V (k = 64 keys) into
//                      the output accumulator, which stays in tensor memory for the whole block,
//                      with P read from tensor memory and V as the M/N-contiguous operand it is;
//   warps 0-3          one thread per query row (its lane of tensor memory): read the row of S with
//                      tcgen05.ld (one round trip), its maximum without any shuffle, P = 2^(s - m) rounded to
//                      bfloat16 and written BACK INTO TENSOR MEMORY with tcgen05.st, two to a column over the first
//                      half of the row of S it came from; P V takes its A operand from there (no shared-memory round
//                      trip, no proxy fence, and the tensor core reads 16 KB less shared memory per tile).  The running
//                      maximum m is only raised when the new one exceeds it by more than 8 (P then stays below 2^8,
//                      harmless in bfloat16 and 32-bit sums); raising it means rescaling the accumulator in tensor
//                      memory (tcgen05.ld, multiply, tcgen05.st), which after the first tiles is rare.  At the end the
//                      row's output is read once and divided by the row sum.
// TWO blocks share an SM (half of its tensor memory each): the softmax of a tile is a chain of latencies
// (tensor-memory load, maxima, exponentials, tensor-memory store) during which a block's own tensor-core work is one
// tile ahead at most; the other block's products and softmax fill the gaps.
//
// Measured at 2048 tokens of 32 heads of 128 (8192 tokens in brackets):
//   one block per SM, 128-key tiles, two threads per row                          57.9 us (621)
//   this form with P through shared memory and a wait, MMAs, commit in turn        44.6 us (530)
//   the same with P in tensor memory                                              43.0 us (510)
//   this form (the issuing thread's work in two blocks of instructions a tile, two commits instead of four)   42.0 us (501)
//   the form before alone on its SM (shared memory padded)                        70.6 us (877)
//   two blocks per SM, two threads per row (sixteen softmax warps exchanging maxima)   53.5 us
//   the probabilities taken with the standing maximum, beside the search for the new one   45.3 us (against 43.0)
//   with the key and value waits skipped when a question asked a tile ahead said yes: 41.2 us (494), withdrawn (see the issuer)
//   the same with the softmax threads' question about the next S asked a tile ahead        41.5 us
//   256 rows to a block alone on its SM: two query tiles A and B that share every key and value tile, key tiles of
//   128, S_A S_B O_A O_B filling tensor memory, P over S, one softmax group per query tile working while the tensor
//   core does the other tile's products                                          52.2 us (560) (against 43.0)
// Notes taken with the SM's clock inside the roles said where a tile's 1950 cycles went in the form with 43.0 us.  The
// issuing thread was never idle in them: about 800 until the eight MMAs of S were accepted, 520 for the four of P V,
// 420 in three waits that succeeded at once, 200 around the loop; `probe_mma_rate` then showed that such a thread
// pays 45 cycles per MMA, 170 per commit and 190 per wait whose answer it reads at once, while the tensor core
// itself takes its nominal 32 cycles for 128 x 64 x 16 (see the issuer below for what was done about it).  A softmax
// thread needs about 1500 cycles a tile for its own chain (wait and load 260, maxima 290, exponentials 650 to 990,
// store and arrive 100), the SM's exponential unit is busy for 1024 of them, and with the issuer out of the way that
// chain is what a tile costs.  The profiler's counters: tensor pipe 39 % active, issue slots 43 % used, the tensor
// core's operand reads 35 % of the shared-memory data pipe: no unit is full.  The form with 256 rows reads Q once per
// 128 keys, but each query tile's chain there is serial (its S is single: softmax 2000 cycles, then P V and the next
// S), so it ends at 4400 cycles per tile of 128 keys for both query tiles, no better per key.  A prompt of 512
// tokens has too few blocks for two per SM and pays for the short tiles: 12.3 us against 10.5.
// Softmax statistics, the accumulator and the final division are 32-bit.
//
// Every mbarrier wait is bounded; on expiry a code goes to status[0] and the block drains.
#include "tc_common.cuh"

RL_DEFINE_ERROR_TEXT()

#define BMQ 128          // query rows per block
#define BNK 64           // keys per tile = one cache page
#define PAGE 64
#define KV_STAGES 2          // (two, like the S buffers: the kernel uses one barrier for "S complete" and "key stage free")
#define SUBQ_BYTES (128 * 64 * 2)       // a [128 rows][64 columns] swizzled sub-tile of Q: 16 KB
#define SUBK_BYTES (64 * 64 * 2)        // a [64 keys][64 dims] swizzled sub-tile of K or V: 8 KB
#define SOFTMAX_WARPS 4
#define NUM_THREADS ((SOFTMAX_WARPS + 2) * 32)
#define TMEM_COLS 256                   // S0 at 0, S1 at 64, O at 128
#define O_COL 128
#define RESCALE_THRESHOLD 8.0f          // in base-2 exponents
#define SMALL_BYTES 512
// Q is HD / 64 sub-tiles of 16 KB; a K or V tile HD / 64 sub-tiles of 8 KB.  Two blocks must fit an SM and
// no more (a third would wait for tensor memory): at head size 64 the request is padded to that end.
#define SMEM_NEEDED(HD) ((HD) / 64 * SUBQ_BYTES + 2 * KV_STAGES * ((HD) / 64) * SUBK_BYTES + SMALL_BYTES)
#define SMEM_BYTES_OF(HD) (SMEM_NEEDED(HD) > 80 * 1024 ? SMEM_NEEDED(HD) : 80 * 1024)

struct SmallItems {
  uint64_t q_full, k_full[KV_STAGES], v_full[KV_STAGES];
  uint64_t s_full[2], p_ready, pv_done[2];
  uint64_t drain_bar;              // an issuer that gives up waits here for the MMAs it has issued
  uint32_t tmem_slot;
  int abort_flag;
};
static_assert(sizeof(SmallItems) <= SMALL_BYTES, "the small items must fit behind the tiles");
static_assert(KV_STAGES == 2, "tile j's key / value stage and its S buffer / product barrier share the index j & 1");
static_assert(SOFTMAX_WARPS * ROW_STAGE_BYTES <= SUBQ_BYTES, "the output's way out uses the queries' buffer");
static_assert(2 * (SMEM_BYTES_OF(128) + 1024) <= 228 * 1024, "two blocks must fit an SM's shared memory");

// 2^x for x <= 8 or so; -inf gives 0
__device__ __forceinline__ float exp2_fast(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// The MMAs of S = Q K^T for one key tile (a k step is 16 dims; Q and K lie in sub-tiles of 64 dims: 16 KB and 8 KB
// apart, in the descriptors' units of 16 bytes 1024 and 512), their commit, and a question about another barrier asked
// first and read last.  Returns 1 if that barrier's phase `peek_parity` is complete.
template <int HD>
__device__ __forceinline__ uint32_t qk_block(uint32_t tmem_s, uint64_t q_desc, uint64_t k_desc, uint32_t idesc, uint32_t commit_bar,
                                             uint32_t peek_bar, uint32_t peek_parity) {
  uint32_t ready;
  if (HD == 128) {
    asm volatile(
        "{\n"
        ".reg .pred t, f, q;\n"
        ".reg .b64 a1, a2, a3, a4, a5, a6, a7, b1, b2, b3, b4, b5, b6, b7;\n"
        "mbarrier.test_wait.parity.shared::cta.b64 q, [%6], %7;\n"
        "setp.eq.b32 t, 0, 0;\n"
        "setp.ne.b32 f, 0, 0;\n"
        "add.u64 a1, %2, 2;\n"
        "add.u64 b1, %3, 2;\n"
        "add.u64 a2, %2, 4;\n"
        "add.u64 b2, %3, 4;\n"
        "add.u64 a3, %2, 6;\n"
        "add.u64 b3, %3, 6;\n"
        "add.u64 a4, %2, 1024;\n"
        "add.u64 b4, %3, 512;\n"
        "add.u64 a5, %2, 1026;\n"
        "add.u64 b5, %3, 514;\n"
        "add.u64 a6, %2, 1028;\n"
        "add.u64 b6, %3, 516;\n"
        "add.u64 a7, %2, 1030;\n"
        "add.u64 b7, %3, 518;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%1], %2, %3, %4, f;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%1], a1, b1, %4, t;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%1], a2, b2, %4, t;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%1], a3, b3, %4, t;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%1], a4, b4, %4, t;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%1], a5, b5, %4, t;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%1], a6, b6, %4, t;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%1], a7, b7, %4, t;\n"
        "tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%5];\n"
        "selp.u32 %0, 1, 0, q;\n"
        "}\n"
        : "=r"(ready)
        : "r"(tmem_s), "l"(q_desc), "l"(k_desc), "r"(idesc), "r"(commit_bar), "r"(peek_bar), "r"(peek_parity)
        : "memory");
  } else {
    asm volatile(
        "{\n"
        ".reg .pred t, f, q;\n"
        ".reg .b64 a1, a2, a3, b1, b2, b3;\n"
        "mbarrier.test_wait.parity.shared::cta.b64 q, [%6], %7;\n"
        "setp.eq.b32 t, 0, 0;\n"
        "setp.ne.b32 f, 0, 0;\n"
        "add.u64 a1, %2, 2;\n"
        "add.u64 b1, %3, 2;\n"
        "add.u64 a2, %2, 4;\n"
        "add.u64 b2, %3, 4;\n"
        "add.u64 a3, %2, 6;\n"
        "add.u64 b3, %3, 6;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%1], %2, %3, %4, f;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%1], a1, b1, %4, t;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%1], a2, b2, %4, t;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%1], a3, b3, %4, t;\n"
        "tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%5];\n"
        "selp.u32 %0, 1, 0, q;\n"
        "}\n"
        : "=r"(ready)
        : "r"(tmem_s), "l"(q_desc), "l"(k_desc), "r"(idesc), "r"(commit_bar), "r"(peek_bar), "r"(peek_parity)
        : "memory");
  }
  return ready;
}
// The same for O (+)= P V: four MMAs of 16 keys each, P from tensor memory (8 columns a step), V as the M/N-contiguous
// operand (2048 bytes = 128 units a step).
template <int HD>
__device__ __forceinline__ uint32_t pv_block(uint32_t tmem_o, uint32_t tmem_p, uint64_t v_desc, uint32_t idesc, uint32_t accumulate_first,
                                             uint32_t commit_bar, uint32_t peek_bar, uint32_t peek_parity) {
  uint32_t ready;
  asm volatile(
      "{\n"
      ".reg .pred t, p, q;\n"
      ".reg .b64 b1, b2, b3;\n"
      ".reg .b32 a1, a2, a3;\n"
      "mbarrier.test_wait.parity.shared::cta.b64 q, [%7], %8;\n"
      "setp.eq.b32 t, 0, 0;\n"
      "setp.ne.b32 p, %5, 0;\n"
      "add.u32 a1, %2, 8;\n"
      "add.u64 b1, %3, 128;\n"
      "add.u32 a2, %2, 16;\n"
      "add.u64 b2, %3, 256;\n"
      "add.u32 a3, %2, 24;\n"
      "add.u64 b3, %3, 384;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%1], [%2], %3, %4, p;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%1], [a1], b1, %4, t;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%1], [a2], b2, %4, t;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%1], [a3], b3, %4, t;\n"
      "tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%6];\n"
      "selp.u32 %0, 1, 0, q;\n"
      "}\n"
      : "=r"(ready)
      : "r"(tmem_o), "r"(tmem_p), "l"(v_desc), "r"(idesc), "r"(accumulate_first), "r"(commit_bar), "r"(peek_bar), "r"(peek_parity)
      : "memory");
  return ready;
}

template <int HD>
__global__ void __launch_bounds__(NUM_THREADS, 2)
flash_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                        const __grid_constant__ CUtensorMap map_v, const int* __restrict__ block_table, int table_width,
                        const int* __restrict__ seq_start, const int* __restrict__ seq_pos0, bf16* __restrict__ out,
                        int out_stride, int H, int K, int window, float scale_log2, int* __restrict__ status,
                        int test_role, uint32_t test_ns) {
  // All shared memory is dynamic, so that the tiles start at the block's first byte (1024-byte
  // aligned, as the 128-byte swizzle needs) and the small items fit behind them.
  constexpr int SUBS = HD / 64, Q_BYTES = SUBS * SUBQ_BYTES, KV_BYTES = SUBS * SUBK_BYTES;
  extern __shared__ __align__(1024) unsigned char smem_dyn[];
  unsigned char* q_s = smem_dyn;                           // 128 rows x HD
  unsigned char* k_s = q_s + Q_BYTES;                      // KV_STAGES x (64 keys x HD)
  unsigned char* v_s = k_s + KV_STAGES * KV_BYTES;         // KV_STAGES x (64 keys x HD)
  SmallItems& sm = *reinterpret_cast<SmallItems*>(v_s + KV_STAGES * KV_BYTES);
  uint64_t& q_full = sm.q_full;
  uint64_t(&k_full)[KV_STAGES] = sm.k_full;
  uint64_t(&v_full)[KV_STAGES] = sm.v_full;
  uint64_t(&s_full)[2] = sm.s_full;
  uint64_t& p_ready = sm.p_ready;
  uint64_t(&pv_done)[2] = sm.pv_done;
  uint64_t& drain_bar = sm.drain_bar;
  uint32_t& tmem_slot = sm.tmem_slot;
  int& abort_flag = sm.abort_flag;
  if (smem_u32(smem_dyn) & 1023u) {  // uniform over the block; nothing has been set up yet
    if (threadIdx.x == 0) give_up_code(status, 23);
    return;
  }
  const WaitCtl ctl = {&abort_flag, test_role, test_ns};
  int issued_k = 0, issued_v = 0;  // (the producer's lane) key and value tiles whose copies were started

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int s = blockIdx.x / H, h = blockIdx.x % H;
  const int tok0 = seq_start[s];
  const int q_len = seq_start[s + 1] - tok0;
  // Late row tiles have the most keys to visit.  Blocks are handed out in the order of blockIdx.x, then y:
  // with the row tile in y, the last row tiles of ALL heads and sequences go out first, then the ones before,
  // and the short tiles fill the gaps at the end.
  const int row0 = (int)(gridDim.y - 1 - blockIdx.y) * BMQ;
  if (row0 >= q_len) return;  // before any barrier or tensor-memory use: the whole block leaves
  const int pos0 = seq_pos0[s];
  const int kh = h / (H / K);
  const int rows_here = min(BMQ, q_len - row0);
  const int first_pos = pos0 + row0, last_pos = first_pos + rows_here - 1;
  const int lowest_key = (window != 0 && first_pos + 1 > window) ? first_pos + 1 - window : 0;
  const int tile_lo = lowest_key / BNK, tile_hi = last_pos / BNK;
  const int n_tiles = tile_hi - tile_lo + 1;

  if (threadIdx.x == 0) {
    mbar_init(&q_full, 1);
    for (int i = 0; i < KV_STAGES; ++i) {
      mbar_init(&k_full[i], 1);
      mbar_init(&v_full[i], 1);
    }
    mbar_init(&s_full[0], 1);
    mbar_init(&s_full[1], 1);
    mbar_init(&p_ready, SOFTMAX_WARPS);  // one arrival per softmax warp
    mbar_init(&pv_done[0], 1);
    mbar_init(&pv_done[1], 1);
    mbar_init(&drain_bar, 1);
    abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == SOFTMAX_WARPS + 1) tmem_alloc(&tmem_slot, TMEM_COLS);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_slot;
  // barriers and tensor memory are set up: from here on the kernel reads what its predecessor wrote
  pdl_trigger();
  pdl_wait();

  if (warp == SOFTMAX_WARPS) {
    // ---------------- TMA producer
    if (lane == 0) {
      mbar_expect_tx(&q_full, Q_BYTES);
#pragma unroll
      for (int b = 0; b < SUBS; ++b) tma_load_2d(q_s + b * SUBQ_BYTES, &map_q, &q_full, h * HD + 64 * b, tok0 + row0);
      const int* table = block_table + (size_t)s * table_width;
      for (int j = 0; j < n_tiles; ++j) {
        const int st = j % KV_STAGES;
        const uint32_t round = j / KV_STAGES;
        const int tile = tile_lo + j;
        const int page = tile < table_width ? table[tile] : 0;  // a page past the sequence's end is never attended to
        // K
        // (a key stage is free when the S it fed is complete, a value stage when its P V is: with two stages and two S
        // buffers, tile j's stage and its S buffer have the same index, and one commit serves both waiters)
        if (round > 0 && !mbar_wait_role(&s_full[st], (round - 1) & 1, ctl, 11)) {
          give_up_code(status, 11);
          abort_flag = 1;
          break;
        }
        if (*(volatile int*)&abort_flag) break;
        mbar_expect_tx(&k_full[st], KV_BYTES);
#pragma unroll
        for (int b = 0; b < SUBS; ++b) tma_load_4d(k_s + (size_t)st * KV_BYTES + b * SUBK_BYTES, &map_k, &k_full[st], 64 * b, 0, kh, page);
        issued_k = j + 1;
        // V
        if (round > 0 && !mbar_wait_role(&pv_done[st], (round - 1) & 1, ctl, 12)) {
          give_up_code(status, 12);
          abort_flag = 1;
          break;
        }
        mbar_expect_tx(&v_full[st], KV_BYTES);
#pragma unroll
        for (int b = 0; b < SUBS; ++b) tma_load_4d(v_s + (size_t)st * KV_BYTES + b * SUBK_BYTES, &map_v, &v_full[st], 64 * b, 0, kh, page);
        issued_v = j + 1;
      }
    }
  } else if (warp == SOFTMAX_WARPS + 1) {
    // ---------------- tensor-core issuer
    if (lane == 0) {
      const uint32_t idesc_qk = make_idesc_bf16(BMQ, BNK, 0, 0);
      const uint32_t idesc_pv = make_idesc_bf16(BMQ, HD, 0, 1);
      const uint32_t q_addr = smem_u32(q_s);
      bool ok = mbar_wait_role(&q_full, 0, ctl, 13);
      if (!ok) {
        give_up_code(status, 13);
        abort_flag = 1;
      }
      // Everything this thread asks of the barriers costs it a round trip when it reads the answer at once (190
      // cycles for a wait that succeeds, 170 for a commit, 45 for an MMA: measured with `probe_mma_rate`), and twelve
      // MMAs, four commits and three waits a tile kept it busy for all of a tile's 1950 cycles.  So a tile's products
      // go out as two blocks of instructions (qk_block, pv_block), each with ONE commit.  Each block also asks about
      // data that is needed later (mbarrier.test_wait, before its MMAs, read after them); the answers are NOT used
      // to skip the waits below: the tensor-core GEMM's issuer, built the same way, gave up on a stage about once in
      // 10^5 launches when it skipped its wait after a yes, and until that is understood every tile is waited for.
      const uint64_t q_desc = make_smem_desc(q_addr);
      uint32_t v_ready = 0, k_ready = 0;  // the answers: value tile j, key tile j + 2 (for the S after next) have landed
      auto wait_for = [&](uint64_t* bar, uint32_t parity, int code) -> bool {
        if (mbar_wait_role(bar, parity, ctl, code)) return true;
        give_up_code(status, code);
        abort_flag = 1;
        return false;
      };
      // S(j) = Q K(j)^T into S buffer j & 1; asks for value tile `jv` (used by the P V that comes next)
      auto issue_qk = [&](int j, int jv) {
        const int st = j % KV_STAGES;
        tc_fence_after();
        v_ready = qk_block<HD>(tmem_base + (uint32_t)((j & 1) * BNK), q_desc, make_smem_desc(smem_u32(k_s + (size_t)st * KV_BYTES)), idesc_qk,
                               smem_u32(&s_full[j & 1]), smem_u32(&v_full[jv % KV_STAGES]), (uint32_t)((jv / KV_STAGES) & 1));
      };
      if (ok) ok = wait_for(&k_full[0], 0, 14);
      if (ok) issue_qk(0, 0);
      if (ok && n_tiles > 1) {
        ok = wait_for(&k_full[1], 0, 14);
        if (ok) issue_qk(1, 0);
      }
      for (int j = 0; j < n_tiles && ok; ++j) {
        // S of tile j + 1 was issued before this tile's softmax began (above, or at the end of the trip before).  Its
        // buffer was last read by the P V of tile j - 1, which stands before it in this thread's order.
        if (!(ok = wait_for(&p_ready, j & 1, 15))) break;
        const int st = j % KV_STAGES;
        if (!(ok = wait_for(&v_full[st], (j / KV_STAGES) & 1, 16))) break;
        tc_fence_after();
        // O += P(j) V(j); asks for key tile j + 2
        const int jk = j + 2;
        k_ready = pv_block<HD>(tmem_base + O_COL, tmem_base + (uint32_t)((j & 1) * BNK),
                               make_smem_desc_mn(smem_u32(v_s + (size_t)st * KV_BYTES), SUBK_BYTES, 1024), idesc_pv, j > 0 ? 1u : 0u,
                               smem_u32(&pv_done[j & 1]), smem_u32(&k_full[jk % KV_STAGES]), (uint32_t)((jk / KV_STAGES) & 1));
        if (jk < n_tiles) {
          // S of tile j + 2 goes into the buffer whose P this product has just been told to read
          if (!(ok = wait_for(&k_full[jk % KV_STAGES], (jk / KV_STAGES) & 1, 14))) break;
          issue_qk(jk, j + 1);
        } else {
          v_ready = 0;  // (nobody asked about value tile j + 1)
        }
      }
      if (*(volatile int*)&abort_flag) {
        // the tensor core may still be at work on what was issued before a wait failed: tensor memory is not
        // given back, and the block does not end, before that is done (bounded like the drain)
        umma_commit(&drain_bar);
        mbar_wait(&drain_bar, 0);
      }
    }
  } else {
    // ---------------- softmax and output: warp w owns tensor-memory lanes 32 w .. 32 w + 31, one thread a query row
    const int r = warp * 32 + lane;
    const int qpos = first_pos + r;
    const uint32_t lane_addr = tmem_base + ((uint32_t)(warp * 32) << 16);
    const uint32_t o_addr = lane_addr + O_COL;
    float m_run = -INFINITY, l_run = 0.f;   // m_run in units of raw scores times scale_log2
    bool ok = true;
    auto give_up = [&](int code) {
      if (lane == 0) {
        give_up_code(status, code);
        abort_flag = 1;
      }
      ok = false;
    };
    for (int j = 0; j < n_tiles && ok; ++j) {
      if (!mbar_wait_role(&s_full[j & 1], (j >> 1) & 1, ctl, 17)) {
        give_up(17);
        break;
      }
      if (*(volatile int*)&abort_flag) {
        ok = false;
        break;
      }
      tc_fence_after();
      const int key0 = (tile_lo + j) * BNK;
      const bool need_mask = key0 + BNK - 1 > first_pos || window != 0;
      const uint32_t s_addr = lane_addr + (uint32_t)((j & 1) * BNK);
      // this thread's row of S in one round trip
      uint32_t v[BNK];
#pragma unroll
      for (int c = 0; c < BNK / 32; ++c) tmem_ld_32x32b_x32(s_addr + c * 32, *reinterpret_cast<uint32_t(*)[32]>(&v[c * 32]));
      tmem_ld_wait();
      // (four running maxima and, below, four running sums: one chain of 64 dependent operations would leave the
      // few warps of an SM waiting on their own arithmetic)
      float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
      if (need_mask) {
#pragma unroll
        for (int i = 0; i < BNK; ++i) {
          const int key = key0 + i;
          if (key > qpos || (window != 0 && qpos - key >= window)) v[i] = __float_as_uint(-INFINITY);
          mx4[i & 3] = fmaxf(mx4[i & 3], __uint_as_float(v[i]));
        }
      } else {
#pragma unroll
        for (int i = 0; i < BNK; ++i) mx4[i & 3] = fmaxf(mx4[i & 3], __uint_as_float(v[i]));
      }
      float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
      mx *= scale_log2;   // the scale is positive: the maximum commutes with it
      // raise the running maximum only when it pays (see the header); the first tile sets it
      const bool raise = mx > m_run + RESCALE_THRESHOLD || (m_run == -INFINITY && mx != -INFINITY);
      const float m_next = raise ? mx : m_run;
      const float a = (raise && m_run != -INFINITY) ? exp2f(m_run - m_next) : 1.0f;
      const bool rescale = j > 0 && __any_sync(0xffffffffu, raise && m_run != -INFINITY);
      m_run = m_next;
      const float neg_m = (m_run == -INFINITY) ? 0.f : -m_run;  // a row past the sequence's end may see nothing
      if (rescale) {
        // the accumulator holds sums scaled by 2^-m_run(old): bring this warp's rows to 2^-m_next, once the product
        // of the tile before is done
        if (!mbar_wait_role(&pv_done[(j - 1) & 1], ((j - 1) >> 1) & 1, ctl, 18)) {
          give_up(18);
          break;
        }
        tc_fence_after();
#pragma unroll 1
        for (int c = 0; c < HD / 32; ++c) {
          uint32_t o[32];
          tmem_ld_32x32b_x32(o_addr + c * 32, o);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * a);
          tmem_st_32x32b_x32(o_addr + c * 32, o);
        }
      }
      // The probabilities, rounded to bfloat16, go back into tensor memory two to a column, over the first half of
      // this row of S, and the product reads them there.  (The S buffer's next product comes after this tile's P V in
      // the issuing thread's order, and the tensor core keeps that order.)
      uint32_t pk[BNK / 2];
      float sum4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int i = 0; i < BNK / 2; ++i) {
        const float p0 = exp2_fast(fmaf(__uint_as_float(v[2 * i]), scale_log2, neg_m));
        const float p1 = exp2_fast(fmaf(__uint_as_float(v[2 * i + 1]), scale_log2, neg_m));
        sum4[i & 3] += p0 + p1;
        pk[i] = pack2(p0, p1);
      }
      tmem_st_32x32b_x32(s_addr, pk);
      l_run = l_run * a + ((sum4[0] + sum4[1]) + (sum4[2] + sum4[3]));
      tmem_st_wait();
      // P is complete (and the accumulator rescaled if it had to be): hand both to the tensor core
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_ready);
    }
    if (ok && !mbar_wait_role(&pv_done[(n_tiles - 1) & 1], ((n_tiles - 1) >> 1) & 1, ctl, 20)) give_up(20);
    ok = __all_sync(0xffffffffu, ok);  // (the way out below works as a warp)
    if (ok) {
      tc_fence_after();
      const float inv = l_run > 0.f ? 1.0f / l_run : 0.f;
      // This thread holds a row of the output; the warp turns 64 dims of its 32 rows at a time through the
      // queries' buffer, which no product reads any more, and writes whole 128-byte rows (see tc_common.cuh).
      const uint32_t stage = smem_u32(q_s) + (uint32_t)(warp * ROW_STAGE_BYTES);
      const int rows_valid = rows_here - warp * 32;  // (may be <= 0: nothing is written then)
      bf16* o = out + (size_t)(tok0 + row0 + warp * 32) * out_stride + (size_t)h * HD;
#pragma unroll 1
      for (int c = 0; c < HD / 64; ++c) {
        uint32_t v0[32], v1[32];
        tmem_ld_32x32b_x32(o_addr + c * 64, v0);
        tmem_ld_32x32b_x32(o_addr + c * 64 + 32, v1);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          v0[i] = __float_as_uint(__uint_as_float(v0[i]) * inv);
          v1[i] = __float_as_uint(__uint_as_float(v1[i]) * inv);
        }
        store_rows64_bf16(o + c * 64, out_stride, rows_valid, v0, v1, stage, lane);
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == SOFTMAX_WARPS + 1) tmem_dealloc(tmem_base, TMEM_COLS);
  // Every role is done or has given up.  Nothing may still be writing shared memory when the block ends: if
  // someone gave up, the producer's lane waits (bounded, with the long limit) for the copies that were
  // started.  It does so here, after the roles have met, because it may have left its loop before another
  // role gave up.
  if (threadIdx.x == SOFTMAX_WARPS * 32 && *(volatile int*)&abort_flag) {
    mbar_wait(&q_full, 0);
    for (int j = max(0, issued_k - KV_STAGES); j < issued_k; ++j) mbar_wait(&k_full[j % KV_STAGES], (j / KV_STAGES) & 1);
    for (int j = max(0, issued_v - KV_STAGES); j < issued_v; ++j) mbar_wait(&v_full[j % KV_STAGES], (j / KV_STAGES) & 1);
  }
}

// ------------------------------------------------------------------ host side
// Head sizes this kernel is built for: 64 and 128 (1 if `hd` is one of them).
RL_API int rl_flash_prefill_tc_takes(int hd) { return hd == 64 || hd == 128; }

template <int HD>
static int launch_flash_tc(const void* q, int q_stride, int n_tokens, const void* k_pages, const void* v_pages, int n_pages,
                           const int* block_table, int table_width, const int* seq_start, const int* seq_pos0, void* out,
                           int out_stride, int n_seqs, int max_q_len, int H, int K, int window, float scale, int* status,
                           int wait_test_role, unsigned int wait_test_ns, cudaStream_t stream) {
  CUtensorMap map_q, map_k, map_v;
  if (make_matrix_map(&map_q, q, n_tokens, q_stride, q_stride, BMQ))
    RL_REFUSE(10, "flash_prefill_tc: cannot describe the query tensor to TMA");
  if (make_page_map(&map_k, k_pages, n_pages, K, PAGE, HD, PAGE) || make_page_map(&map_v, v_pages, n_pages, K, PAGE, HD, PAGE))
    RL_REFUSE(11, "flash_prefill_tc: cannot describe the cache pages to TMA");
  const size_t smem = SMEM_BYTES_OF(HD);
  auto kern = flash_prefill_tc_kernel<HD>;
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
    RL_REFUSE(12, "flash_prefill_tc: cannot get %zu bytes of shared memory", smem);
  dim3 grid(H * n_seqs, (max_q_len + BMQ - 1) / BMQ);
  RL_LAUNCH_CHECK(rl_launch(kern, grid, NUM_THREADS, smem, stream, map_q, map_k, map_v, block_table, table_width, seq_start, seq_pos0,
                            (bf16*)out, out_stride, H, K, window, scale * 1.4426950408889634f, status, wait_test_role,
                            (uint32_t)wait_test_ns));
  return 0;
}

// status: one int in device memory, 0 before the call; afterwards non-zero means that a bounded wait
// expired (11, 12 the producer for a free key / value stage; 13, 14, 15, 16 the tensor-core issuer for the
// queries, a key tile, the probabilities, a value tile; 17, 18, 20 a softmax warp for the scores, the product before
// a rescale, the last product; 23: shared memory not aligned)
// and the output is not valid.  wait_test_role, wait_test_ns: 0, 0 in normal use; a test names one of these
// codes and a limit in nanoseconds, and that role's waits give up after that long instead of a second.
RL_API int rl_flash_prefill_tc(const void* q, int q_stride, int n_tokens, const void* k_pages, const void* v_pages,
                               int n_pages, const int* block_table, int table_width, const int* seq_start,
                               const int* seq_pos0, void* out, int out_stride, int n_seqs, int max_q_len, int H, int K,
                               int hd, int page_size, int window, float scale, int* status, int wait_test_role,
                               unsigned int wait_test_ns, cudaStream_t stream) {
  if (n_seqs <= 0 || max_q_len <= 0 || H <= 0 || K <= 0 || n_tokens <= 0 || n_pages <= 0)
    RL_REFUSE(1, "flash_prefill_tc: S=%d max_q=%d H=%d K=%d T=%d pages=%d", n_seqs, max_q_len, H, K, n_tokens, n_pages);
  if (!rl_flash_prefill_tc_takes(hd)) RL_REFUSE(2, "flash_prefill_tc: head size %d, this kernel is built for 64 and 128", hd);
  if (H % K) RL_REFUSE(3, "flash_prefill_tc: %d query heads are not a multiple of %d kv heads", H, K);
  if (page_size != PAGE) RL_REFUSE(4, "flash_prefill_tc: page size %d, this kernel is built for %d", page_size, PAGE);
  if (q_stride % 8 || out_stride % 8) RL_REFUSE(5, "flash_prefill_tc: strides %d/%d break 16-byte alignment", q_stride, out_stride);
  if (((uintptr_t)q | (uintptr_t)k_pages | (uintptr_t)v_pages | (uintptr_t)out) & 15) RL_REFUSE(6, "flash_prefill_tc: operands must be 16-byte aligned");
  if ((long long)H * n_seqs > 0x7fffffffLL || (max_q_len + BMQ - 1) / BMQ > 65535)
    RL_REFUSE(7, "flash_prefill_tc: H=%d x S=%d blocks or %d query rows exceed the grid", H, n_seqs, max_q_len);
  if (window < 0 || status == nullptr || !(scale > 0.f)) RL_REFUSE(8, "flash_prefill_tc: bad window or scale, or no status word");
  if (hd == 64)
    return launch_flash_tc<64>(q, q_stride, n_tokens, k_pages, v_pages, n_pages, block_table, table_width, seq_start, seq_pos0, out,
                               out_stride, n_seqs, max_q_len, H, K, window, scale, status, wait_test_role, wait_test_ns, stream);
  return launch_flash_tc<128>(q, q_stride, n_tokens, k_pages, v_pages, n_pages, block_table, table_width, seq_start, seq_pos0, out,
                              out_stride, n_seqs, max_q_len, H, K, window, scale, status, wait_test_role, wait_test_ns, stream);
}
