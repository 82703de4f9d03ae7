// sm_100a building blocks shared by the tcgen05 kernels: mbarrier with bounded waits,
// shared-memory matrix descriptors, tcgen05.mma / commit / alloc / ld wrappers, and the
// 3xTF32 operand split.  Everything here is inline PTX written for this library.
#pragma once
#include <cuda_runtime.h>
#include <cstdint>

namespace b200 {
namespace tc {

// Device status word (global memory owned by the runtime, passed to every kernel): 0 = fine;
// otherwise (code << 24 | CTA index) of the first bounded wait that gave up.  Read by the host
// after a synchronise (b200_device_status).

constexpr int STATUS_TIMEOUT_FULL = 1;   // MMA warp: operands never arrived
constexpr int STATUS_TIMEOUT_EMPTY = 2;  // producer: stage never released
constexpr int STATUS_TIMEOUT_ACCUM = 3;  // epilogue: accumulator never completed
constexpr int STATUS_TIMEOUT_TMA = 4;    // bulk copy never landed

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ unsigned long long global_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}

// ---- mbarrier ----------------------------------------------------------------------------
#ifndef B200_WAIT_HINT_NS
#define B200_WAIT_HINT_NS 1000
#endif
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
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
// The same with a suspend-time hint: the hardware may park the thread for up to `ns` nanoseconds
// and wakes it when the phase completes.  Waiting warps then stay out of the shared-memory pipe,
// which the working roles of the CTA (epilogue stores, producer stores) need.
__device__ __forceinline__ bool mbar_try_hint(uint32_t bar, uint32_t parity, uint32_t ns) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity), "r"(ns)
      : "memory");
  return ok != 0;
}
// Wait with a wall-clock bound.  On expiry the status word and the CTA's abort flag are set and
// false is returned; every role then falls through to the common teardown (TMEM is freed, the
// kernel returns, the context stays usable).  Other waiters notice the abort flag and leave too.
constexpr uint32_t WAIT_HINT_NS = B200_WAIT_HINT_NS;
constexpr unsigned long long WAIT_LIMIT_NS = 2000000000ull;  // 2 s: no legitimate wait is near this
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int* status,
                                          int code) {
  if (mbar_try(bar, parity)) return true;
  unsigned long long t0 = 0;
  uint32_t spins = 0;
  while (!mbar_try_hint(bar, parity, WAIT_HINT_NS)) {
    if (((++spins) & 63u) == 0) {
      if (abort_flag && *abort_flag) return false;
      const unsigned long long now = global_ns();
      if (t0 == 0) t0 = now;
      else if (now - t0 > WAIT_LIMIT_NS) {
        atomicCAS(status, 0, (code << 24) | (int)(blockIdx.x & 0xFFFFFF));
        if (abort_flag) *abort_flag = 1;
        return false;
      }
    }
  }
  return true;
}
// One lane of a converged warp (the same lane every time), for instructions that a single thread must issue
// while the warp's control flow stays uniform.
__device__ __forceinline__ bool elect_one() {
  uint32_t is_leader;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "elect.sync _|p, 0xffffffff;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(is_leader));
  return is_leader != 0;
}
// mbar_wait for a whole warp: every lane polls, and the warp leaves together with one answer.
__device__ __forceinline__ bool warp_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int* status, int code) {
  const bool ok = mbar_wait(bar, parity, abort_flag, status, code);
  return __all_sync(0xffffffffu, ok);
}
// Bulk copy global -> shared memory of this CTA; completion is counted in bytes on `bar`
// (pair it with mbar_expect_tx).  Both addresses 16-byte aligned, size a multiple of 16.
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
__device__ __forceinline__ void fence_barrier_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
// Make generic-proxy shared-memory writes visible to the async proxy (tcgen05.mma operand reads).
__device__ __forceinline__ void fence_proxy_async() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// ---- tcgen05 -------------------------------------------------------------------------------
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// One warp allocates `cols` (power of two >= 32) TMEM columns; the base address lands in *slot.
__device__ __forceinline__ void tmem_alloc(uint32_t slot_smem_addr, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(slot_smem_addr), "r"(cols)
               : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}

// Shared-memory matrix descriptor for a K-major operand tile stored with the 128-byte swizzle:
// rows of 128 bytes (32 FP32 along K), 8-row groups 1024 bytes apart, tile base 1024-byte aligned.
__device__ __forceinline__ uint64_t make_kmajor_sw128_desc(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);  // start address, 16-byte units
  d |= (uint64_t)1 << 16;                         // leading byte offset: unused for swizzled K-major
  d |= (uint64_t)(1024u >> 4) << 32;              // stride byte offset between 8-row groups
  d |= (uint64_t)1 << 46;                         // descriptor version of sm_100
  d |= (uint64_t)2 << 61;                         // layout: SWIZZLE_128B
  return d;
}
// kind::tf32, FP32 accumulate, both operands K-major, tile M x N.
__host__ __device__ constexpr uint32_t make_idesc_tf32(int M, int N) {
  return (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}
__device__ __forceinline__ void umma_tf32(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                          uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// kind::f16 with BF16 operands, FP32 accumulate, both operands K-major (K = 16 per instruction).
__host__ __device__ constexpr uint32_t make_idesc_bf16(int M, int N) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}
__device__ __forceinline__ void umma_bf16(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                          uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Arrive on `bar` once every tcgen05.mma issued so far by this thread has completed.
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// 32 lanes x 32 consecutive FP32 columns: thread i of the warp receives lane (base lane + i).
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, float (&v)[32]) {
  uint32_t r[32];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}

// 32 lanes x 16 consecutive FP32 columns (half the registers of tmem_ld32, for epilogues that run inside a loop
// whose state stays live)
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, float (&v)[16]) {
  uint32_t r[16];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}

#ifdef B200_SPLIT_MASK_LO
#define B200_SPLIT_LO(r) __uint_as_float(__float_as_uint(r) & 0xFFFFE000u)
#else
#define B200_SPLIT_LO(r) (r)
#endif
// ---- 3xTF32 split --------------------------------------------------------------------------
// x = hi + lo with hi the TF32 value nearest to x (10 explicit mantissa bits, low 13 bits zero)
// and lo the TF32 truncation of the exact FP32 remainder.  a*b is then evaluated as
// hi_a*hi_b + hi_a*lo_b + lo_a*hi_b with FP32 accumulation: relative error about 2^-21 per product.
// Both parts have zero low mantissa bits, so the result does not depend on how the tensor core
// treats bits beyond TF32.
__device__ __forceinline__ void split_tf32(float x, float& hi, float& lo) {
  const uint32_t u = __float_as_uint(x);
  const uint32_t h = (u + 0x1000u) & 0xFFFFE000u;
  hi = __uint_as_float(h);
  const float rem = x - hi;
  // |hi| = inf or NaN (overflowing round-up, or non-finite input): keep hi alone.
  lo = ((h & 0x7F800000u) == 0x7F800000u) ? 0.f : __uint_as_float(__float_as_uint(rem) & 0xFFFFE000u);
}

// Producer-side split (three instructions per value): same hi; lo is the exact remainder, of which
// the tensor core reads the TF32 bits only.  An operand that rounds up past the largest finite TF32
// value (|x| >= 2^128 - 2^115) or is not finite yields NaN where the full split keeps hi alone.
__device__ __forceinline__ void split_tf32_fast(float x, float& hi, float& lo) {
  hi = __uint_as_float((__float_as_uint(x) + 0x1000u) & 0xFFFFE000u);
  lo = B200_SPLIT_LO(x - hi);
}

// ---- split precision with BF16 cross terms ---------------------------------------------------
// x*w = xh*wh + (xh*wl + xl*wh) + xl*wl with xh = TF32 nearest to x and xl = x - xh.  The first
// product runs as kind::tf32 on the hi planes.  The bracket is 2^-11 of the result, so 8-bit
// operands carry it to 2^-20: it runs as ONE kind::f16 (BF16) product of twice the depth over
// "cross" planes that hold, per 32 channels, [bf16(xh) x32 | bf16(xl) x32] for activations and
// [bf16(wl) x32 | bf16(wh) x32] for weights (a 128-byte row either way).  That is one TF32 pass
// plus one BF16 pass of the same duration per K block instead of three TF32 passes.
#ifndef B200_CROSS_BF16
#define B200_CROSS_BF16 1
#endif
constexpr bool CROSS_BF16 = B200_CROSS_BF16 != 0;
// two floats -> packed bf16x2 (first argument in the low half = lower address)
__device__ __forceinline__ uint32_t pack_bf16x2(float first, float second) {
  uint32_t r;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(second), "f"(first));
  return r;
}
// Byte offset of bf16 element k (0..63) of `row` in a 128B-swizzled K-major plane.
__device__ __forceinline__ uint32_t sw128_offset_bf16(int row, int k) {
  return (uint32_t)(row * 128 + ((((k >> 3) ^ (row & 7)) << 4) | ((k & 7) << 1)));
}
__device__ __forceinline__ void sts_b32x4(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}
__device__ __forceinline__ void sts_b32x2(uint32_t addr, uint32_t a, uint32_t b) {
  asm volatile("st.shared.v2.b32 [%0], {%1, %2};" ::"r"(addr), "r"(a), "r"(b) : "memory");
}

// Byte offset of element (row, k) inside a 128B-swizzled K-major tile plane (k in [0,32)).
__device__ __forceinline__ uint32_t sw128_offset(int row, int k) {
  return (uint32_t)(row * 128 + ((((k >> 2) ^ (row & 7)) << 4) | ((k & 3) << 2)));
}
__device__ __forceinline__ void sts_f32(uint32_t addr, float v) {
  asm volatile("st.shared.f32 [%0], %1;" ::"r"(addr), "f"(v) : "memory");
}
__device__ __forceinline__ void sts_f32x4(uint32_t addr, float a, float b, float c, float d) {
  asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}

}  // namespace tc
}  // namespace b200
