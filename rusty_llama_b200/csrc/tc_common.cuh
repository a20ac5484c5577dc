// Wrappers around the PTX of the 5th-generation tensor cores and their plumbing, shared by the
// kernels that use them: mbarriers with bounded waits, TMA tile loads, tensor-memory allocation,
// tcgen05.mma / commit / ld, and the shared-memory and instruction descriptors.
//
// Bounded waits.  A role (producer, tensor-core issuer, product or epilogue warp) waits with
// mbar_wait_role: it polls for the role limit (about one second), looks at the block's abort flag
// now and then, and returns false when the limit ran out or another role has given up.  The caller
// then records its code in the status word (the first code sticks), raises the abort flag and lets the
// block drain, so that a mistake in a pipeline ends in an error message instead of a hung GPU.
// mbar_wait is the wait of the drain itself: it keeps a block alive until the copies it started have
// landed, never looks at the abort flag and always has the long limit (a copy that lands in the
// shared memory of a block that has ended is the fault all of this exists to prevent).
// For tests, a launch may name one role code whose waits get another limit (WaitCtl.test_role,
// test_ns): that role then polls without suspending and reads the clock before every poll, so a limit
// of 0 runs out before the first poll and one of a few nanoseconds before any copy can have arrived.
#pragma once

#include <cuda.h>

#include "common.cuh"

#define WAIT_LIMIT_NS 1000000000ull

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ uint64_t global_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
      "selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ bool mbar_test_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n"
      "selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// The drain's wait: false when the barrier did not flip within WAIT_LIMIT_NS.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
  if (mbar_try_wait(bar, parity)) return true;
  // try_wait itself suspends the thread for a while before it answers "not yet", so this is no
  // busy loop (a __nanosleep here was measured to add about a microsecond to every wait); the clock
  // is read every 16 polls
  // (and for the first time only then: a single thread reads it for nothing, but with every thread of a block
  // of 21 warps reading it at the start of every wait a decode step took 1.5 % longer)
  uint64_t t0 = 0;
  for (uint32_t spins = 1;; ++spins) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((spins & 15u) == 0) {
      if (t0 == 0) t0 = global_ns();
      else if (global_ns() - t0 > WAIT_LIMIT_NS) return false;
    }
  }
}

// What a role's waits need to know: the block's abort flag (shared memory) and the launch's test knob.
struct WaitCtl {
  const volatile int* abort;
  int test_role;
  uint32_t test_ns;
};
// A role's wait (see the header): false when its limit ran out or the block is being abandoned.
__device__ __forceinline__ bool mbar_wait_role(uint64_t* bar, uint32_t parity, const WaitCtl& ctl, int role) {
  if (role == ctl.test_role) {
    // polls while the limit lasts: a limit of 0 has run out before the first poll, whatever has arrived
    const uint64_t t0 = global_ns();
    while (global_ns() - t0 < ctl.test_ns)
      if (mbar_test_wait(bar, parity)) return true;
    return false;
  }
  if (mbar_try_wait(bar, parity)) return true;
  uint64_t t0 = 0;
  for (uint32_t spins = 1;; ++spins) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((spins & 15u) == 0) {
      if (*ctl.abort) return false;
      if (t0 == 0) t0 = global_ns();
      else if (global_ns() - t0 > WAIT_LIMIT_NS) return false;
    }
  }
}
// The same for a caller that keeps the barrier's shared-memory address (a loop that adds to it).
__device__ __forceinline__ bool mbar_try_wait_s(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
      "selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ bool mbar_wait_role_s(uint32_t bar, uint32_t parity, const WaitCtl& ctl, int role) {
  if (role != ctl.test_role && mbar_try_wait_s(bar, parity)) return true;
  uint64_t* p = reinterpret_cast<uint64_t*>(__cvta_shared_to_generic(bar));
  return mbar_wait_role(p, parity, ctl, role);
}
__device__ __forceinline__ void mbar_arrive_s(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
// Records why a block gives up: the first code of a launch stays (later ones are consequences of it).
__device__ __forceinline__ void give_up_code(int* status, int code) { atomicCAS(status, 0, code); }

__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, uint64_t* bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(y)
      : "memory");
}

// The same with shared-memory addresses already in hand (a producer's loop adds to them instead of converting pointers).
__device__ __forceinline__ void mbar_expect_tx_s(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void tma_load_2d_s(uint32_t dst, const CUtensorMap* map, uint32_t bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y)
      : "memory");
}

__device__ __forceinline__ void tmem_alloc(uint32_t* slot_in_smem, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(slot_in_smem)), "r"(cols));
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t addr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(addr), "r"(cols));
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n"
      "}\n" ::"r"(tmem_d), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// D[tmem] (+)= A[tmem] . B[smem]: the A operand is read from tensor memory, a row to a lane, two bfloat16 to a
// column (a k step of 16 is 8 columns), so it costs no shared-memory bandwidth.
__device__ __forceinline__ void umma_bf16_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n"
      "}\n" ::"r"(tmem_d), "r"(tmem_a), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// The four MMAs of a 64-wide k slice in one go: operands are k-major with 128-byte rows, so a k step
// of 16 bfloat16 moves both descriptors' address fields (bytes / 16) by 2.  Only the first one's
// accumulate flag varies.  The thread that issues MMAs is alone in feeding the tensor core, and every
// instruction it spends on descriptors or predicates shows up as idle tensor cycles.
#define RL_UMMA_X4(GROUP)                                                                                     \
  asm volatile(                                                                                               \
      "{\n"                                                                                                   \
      ".reg .pred p, t;\n"                                                                                    \
      ".reg .b64 a1, a2, a3, b1, b2, b3;\n"                                                                   \
      "setp.ne.b32 p, %4, 0;\n"                                                                               \
      "setp.eq.b32 t, 0, 0;\n"                                                                                \
      "add.u64 a1, %1, 2;\n"                                                                                  \
      "add.u64 b1, %2, 2;\n"                                                                                  \
      "add.u64 a2, %1, 4;\n"                                                                                  \
      "add.u64 b2, %2, 4;\n"                                                                                  \
      "add.u64 a3, %1, 6;\n"                                                                                  \
      "add.u64 b3, %2, 6;\n"                                                                                  \
      "tcgen05.mma.cta_group::" GROUP ".kind::f16 [%0], %1, %2, %3, p;\n"                                     \
      "tcgen05.mma.cta_group::" GROUP ".kind::f16 [%0], a1, b1, %3, t;\n"                                     \
      "tcgen05.mma.cta_group::" GROUP ".kind::f16 [%0], a2, b2, %3, t;\n"                                     \
      "tcgen05.mma.cta_group::" GROUP ".kind::f16 [%0], a3, b3, %3, t;\n"                                     \
      "}\n" ::"r"(tmem_d), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate_first)                         \
      : "memory")
__device__ __forceinline__ void umma_bf16_x4(uint32_t tmem_d, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate_first) {
  RL_UMMA_X4("1");
}
__device__ __forceinline__ void umma_bf16_x4_pair(uint32_t tmem_d, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate_first) {
  RL_UMMA_X4("2");
}

// A k slice of a GEMM as its issuing thread could send it, in one piece: ask whether the NEXT stage's data has landed
// (mbarrier.test_wait, which never suspends), issue this stage's four MMAs, commit them to this stage's `empty`
// barrier, and only then read the answer.  The thread waits some 190 cycles for the answer of a wait and 170 for a
// commit when it asks and reads in one go (measured with `probe_mma_rate`, which uses this function), on top of 45
// per MMA: 650 cycles for a slice whose products take the tensor core 512.  Asked a slice ahead, the answer arrives
// while the MMAs are issued.  `gemm_tc` issued its slices this way for a while (0.975 instead of 0.785 of the nominal
// rate on a single SM) and went back to wait, issue, commit: see its issuer.
// Returns 1 when the next stage is ready (0: the caller waits for it in the ordinary way).
__device__ __forceinline__ uint32_t umma_bf16_x4_commit_peek(uint32_t tmem_d, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                                             uint32_t accumulate_first, uint32_t empty_bar, uint32_t next_full_bar,
                                                             uint32_t next_parity) {
  uint32_t ready;
  asm volatile(
      "{\n"
      ".reg .pred p, t, q;\n"
      ".reg .b64 a1, a2, a3, b1, b2, b3;\n"
      "mbarrier.test_wait.parity.shared::cta.b64 q, [%7], %8;\n"
      "setp.ne.b32 p, %5, 0;\n"
      "setp.eq.b32 t, 0, 0;\n"
      "add.u64 a1, %2, 2;\n"
      "add.u64 b1, %3, 2;\n"
      "add.u64 a2, %2, 4;\n"
      "add.u64 b2, %3, 4;\n"
      "add.u64 a3, %2, 6;\n"
      "add.u64 b3, %3, 6;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%1], %2, %3, %4, p;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%1], a1, b1, %4, t;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%1], a2, b2, %4, t;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%1], a3, b3, %4, t;\n"
      "tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%6];\n"
      "selp.u32 %0, 1, 0, q;\n"
      "}\n"
      : "=r"(ready)
      : "r"(tmem_d), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate_first), "r"(empty_bar), "r"(next_full_bar), "r"(next_parity)
      : "memory");
  return ready;
}

// The barrier receives one arrival when every tcgen05.mma issued before by this thread has completed.
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ void tmem_ld_32x32b_x32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

__device__ __forceinline__ void tmem_st_32x32b_x32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
        "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]),
        "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]),
        "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// ---- results that a thread holds by the ROW (tcgen05.ld gives a lane one row of the accumulator), on their way out.
// Stores straight from such registers put 16 bytes into each of 32 different lines per instruction.  A warp turns
// its 32 rows x 64 bfloat16 columns through ROW_STAGE_BYTES of shared memory instead (1024-byte aligned; 16-byte
// pieces swizzled by the row, so that neither the row-wise writes nor the line-wise reads conflict) and writes whole
// 128-byte rows, eight lanes to a row.
#define ROW_STAGE_BYTES 4096
__device__ __forceinline__ uint32_t pack2(float a, float b) {
  __nv_bfloat162 p = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&p);
}
// 64 columns of this lane's row (two tensor-memory loads) -> out[rows of the warp][col0 .. col0 + 63]
__device__ __forceinline__ void store_rows64_bf16(bf16* out_tile, int ldo, int rows_valid, const uint32_t (&r0)[32], const uint32_t (&r1)[32],
                                                  uint32_t stage, int lane) {
#pragma unroll
  for (int p = 0; p < 8; ++p) {
    const uint32_t* r = p < 4 ? r0 : r1;
    const int b = (p & 3) * 8;
    const uint32_t x = pack2(__uint_as_float(r[b]), __uint_as_float(r[b + 1])), y = pack2(__uint_as_float(r[b + 2]), __uint_as_float(r[b + 3]));
    const uint32_t z = pack2(__uint_as_float(r[b + 4]), __uint_as_float(r[b + 5])), w = pack2(__uint_as_float(r[b + 6]), __uint_as_float(r[b + 7]));
    asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(stage + lane * 128 + ((p ^ (lane & 7)) << 4)), "r"(x), "r"(y), "r"(z), "r"(w) : "memory");
  }
  __syncwarp();
#pragma unroll
  for (int it = 0; it < 8; ++it) {
    const int rr = it * 4 + (lane >> 3), pc = lane & 7;
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(stage + rr * 128 + ((pc ^ (rr & 7)) << 4)));
    if (rr < rows_valid) *reinterpret_cast<uint4*>(out_tile + (size_t)rr * ldo + pc * 8) = v;
  }
  __syncwarp();
}

// Shared-memory matrix descriptor of a K-major tile whose rows are 128 bytes (64 bf16) and 128-byte
// swizzled, as TMA writes it: start address, stride between 8-row groups = 1024 bytes, descriptor
// version 1, layout type 2 (128-byte swizzle).  The leading-dimension field is not used by this layout.
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3FFFF) >> 4);
  d |= (uint64_t)1 << 16;
  d |= (uint64_t)(1024 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}

// Instruction descriptor of kind::f16: D 32-bit, A and B bfloat16, both K-major, N and M of the tile.
__device__ __forceinline__ uint32_t make_idesc(int m, int n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}


__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ void tma_load_4d(void* dst, const CUtensorMap* map, uint64_t* bar, int c0, int c1, int c2, int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
      ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}

// Writes made with ordinary stores to shared memory become visible to the tensor core and TMA
// (the async proxy) after this fence.
__device__ __forceinline__ void fence_async_shared() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// Descriptor of an operand whose rows (M or N index) are contiguous instead of k: 128-byte rows hold
// 64 consecutive M/N elements of one k, eight k make a 1024-byte swizzle atom, `sbo_bytes` leads to
// the next eight k and `lbo_bytes` to the next 64 M/N elements (128-byte swizzle, as TMA writes a
// [k][64 elements] box).
__device__ __forceinline__ uint64_t make_smem_desc_mn(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3FFFF) >> 4);
  d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFF) << 16;
  d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFF) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}

// kind::f16 instruction descriptor with bfloat16 operands, 32-bit accumulator; a_mn / b_mn: the
// operand's M/N index is the contiguous one (else k is).
__device__ __forceinline__ uint32_t make_idesc_bf16(int m, int n, int a_mn, int b_mn) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)a_mn << 15) | ((uint32_t)b_mn << 16) | ((uint32_t)(n >> 3) << 17) |
         ((uint32_t)(m >> 4) << 24);
}

// ------------------------------------------------------------------ host side
// cuTensorMapEncodeTiled, asked from the driver at run time (the libraries do not link against libcuda).
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_tiled() {
  static EncodeTiledFn fn = nullptr;
  if (fn) return fn;
  void* p = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess)
    return nullptr;
  fn = (EncodeTiledFn)p;
  return fn;
}

// rows x cols bfloat16 matrix with row stride ld (elements): boxes of 64 columns x `box_rows` rows, 128-byte
// swizzled; rows and columns past the matrix arrive as zeros.  0 on success.
static int make_matrix_map(CUtensorMap* map, const void* base, int rows, int cols, int ld, int box_rows) {
  EncodeTiledFn enc = encode_tiled();
  if (!enc) return 1;
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
  cuuint32_t box[2] = {64, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  return enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
             CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS ? 0 : 2;
}

// The 4-D view of a group's cache pages that the attention kernels copy from: [page][kv head][position][dim],
// boxes of 64 dims x `box_rows` positions of one head of one page, 128-byte swizzled.  0 on success.
static int make_page_map(CUtensorMap* map, const void* pages, int n_pages, int kv_heads, int page_size, int head_dim, int box_rows) {
  EncodeTiledFn enc = encode_tiled();
  if (!enc) return 1;
  cuuint64_t dims[4] = {(cuuint64_t)head_dim, (cuuint64_t)page_size, (cuuint64_t)kv_heads, (cuuint64_t)n_pages};
  cuuint64_t strides[3] = {(cuuint64_t)head_dim * 2, (cuuint64_t)page_size * head_dim * 2, (cuuint64_t)kv_heads * page_size * head_dim * 2};
  cuuint32_t box[4] = {64, (cuuint32_t)box_rows, 1, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  return enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(pages), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
             CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS ? 0 : 2;
}
