// Block-scaled GEMM for sm_100a:  D[m, n] = alpha * sum_k A[m, k] * B[n, k]
//
// Both operands are stored with the reduction axis contiguous (FP4: two codes per byte,
// FP8: one byte per element) and carry one scale per 16 (NVFP4, UE4M3) or 32 (MXFP4 /
// MXFP8, UE8M0) elements in the packed layout described in altob200.h.
//
// Structure of one CTA of the single-CTA kernel (352 threads, persistent over output tiles of 128 x BN):
//   warp 0      : producer.  The whole warp runs the loop, one elected lane issues, per k-stage, two
//                 tiled TMA loads (A: 128 rows x 128 bytes, B: BN rows x 128 bytes, 128-byte swizzle)
//                 and the bulk copies of the stage's scale tiles, all completing on the stage's "full"
//                 mbarrier.
//   warp 1      : MMA issuer.  Owns tensor memory (512 columns).  Per stage one elected lane issues
//                 four tcgen05.mma (each consumes 32 bytes of K per row), then commits to the stage's
//                 "empty" mbarrier; after the last stage of a tile it commits to the accumulator's
//                 "full" mbarrier.  It never waits on an mbarrier itself (that leaves the tensor pipe
//                 idle for ~150 cycles per wait): warp 10 does and releases it through a named barrier.
//   warps 6..9  : scale transfer.  Each warp owns one 32-lane quarter of tensor memory and, per stage,
//                 moves the stage's scale tiles shared memory -> registers -> tensor memory
//                 (tcgen05.st), then arrives on the stage's "scales ready" mbarrier.  (A tcgen05.cp in
//                 the MMA issuer's stream costs a pipeline bubble of ~500 cycles per stage.)
//   warps 2..5  : epilogue.  Each warp reads its 32-lane quarter of the accumulator with tcgen05.ld,
//                 multiplies by alpha, converts, writes 32 rows x 128 bytes into a 128-byte-swizzled
//                 staging buffer and hands it to a TMA store (which also clips ragged M/N edges); two
//                 staging buffers per warp keep stores in flight.
//   warp 10     : waits on the stage's barriers on behalf of the MMA issuer.
// The CTA-pair kernel (cta_group::2, 256 x 256 tiles, 512 threads) and the two-level MXFP4 kernel
// (gemm_macro.cuh) have the same roles; their layouts are described at the kernels.
// Every mbarrier wait is bounded by a cycle count; a wait that gives up records {kernel, block, site}
// in a device status word, raises a CTA-wide abort flag, and all roles fall through to the common
// teardown that frees tensor memory.  All kernels are launched with programmatic stream serialisation
// and wait for the kernel in front of them after their set-up (see launch_after in common.cuh).
#include <cuda.h>
#include <stdio.h>
#include <stdlib.h>

#include <atomic>

#include "common.cuh"

namespace altob200 {

__device__ int g_status[4] = {0, 0, 0, 0};

constexpr int BM = 128;
constexpr int STAGE_K_BYTES = 128;
constexpr int NUM_THREADS = 352;  // producer, MMA issuer, 4 epilogue warps, 4 scale-transfer warps, the wait warp
constexpr int NUM_THREADS_PAIR = 512;  // pair kernel: four warpgroups (see the kernel)
constexpr uint64_t WAIT_LIMIT_NS = 4000000000ull;  // default limit of one wait: 4 s

enum { KIND_NVF4 = 0, KIND_MXF4 = 1, KIND_MXF8 = 2 };

template <int KIND>
struct Kind;
template <>
struct Kind<KIND_NVF4> {
  static constexpr int SF_TILES = 4;  // 512-byte scale tiles per 128 rows per stage
  static constexpr int ELEMS_PER_BYTE = 2, BLOCK = 16;
};
template <>
struct Kind<KIND_MXF4> {
  static constexpr int SF_TILES = 2;
  static constexpr int ELEMS_PER_BYTE = 2, BLOCK = 32;
};
template <>
struct Kind<KIND_MXF8> {
  static constexpr int SF_TILES = 1;
  static constexpr int ELEMS_PER_BYTE = 1, BLOCK = 32;
};

struct GemmArgs {
  int64_t M, N, K;       // K in elements
  int64_t k_bytes;       // bytes per operand row
  const uint8_t* sfa;    // packed scales of A
  const uint8_t* sfb;    // packed scales of B (per expert: stride sfb_expert_stride)
  int64_t nct;           // scale tiles per 128-row block = ceil(K / BLOCK / 4)
  const float* alpha_a;
  const float* alpha_b;
  void* d;
  int64_t ldd;
  int out_bf16;
  // grouped mode (num_experts > 0): B rows are [num_experts * N], group_expert[m / 128]
  int num_experts;
  const int32_t* group_expert;
  int64_t sfb_expert_stride;
  // K-range mode (k_offs != NULL): batch entry e reduces over elements [k_offs[e-1], k_offs[e]) of
  // the shared operands and writes D[e] (grouped wgrad); `num_batches` entries, ranges multiples of 128
  const int32_t* k_offs;
  int num_batches;
  int group_m;           // row tiles per raster group (see decode_tile)
  uint32_t idesc[4];    // instruction descriptors of the four MMAs of a stage
  uint64_t wait_ns;     // limit of every mbarrier wait (wall clock)
#ifdef ALTOB200_GEMM_PROFILE
  // profiling switches of a -DALTOB200_GEMM_PROFILE build only (env ALTOB200_GEMM_DEBUG; results are
  // then WRONG): 1 = copy scales only in the first stage of a tile, 2 = skip the global stores, 4 = stop
  // loading operands once the ring is full, 8 = the epilogue returns the accumulator without reading it
  int debug;
#endif
};
#ifdef ALTOB200_GEMM_PROFILE
#define ALTOB200_DBG(a, bit) (((a).debug & (bit)) != 0)
#else
#define ALTOB200_DBG(a, bit) false
#endif

// ---------------------------------------------------------------------------------------
// PTX wrappers
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
#ifdef ALTOB200_WAIT_SPIN
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
#else
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
#endif
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ uint64_t globaltimer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}
// Bounded wait.  Returns false (and raises the abort flag) when the limit passes or when
// another role already aborted.  The limit is counted on the SM's cycle counter (a register
// read); %globaltimer is far too slow to read inside a wait that is on the critical path of
// every pipeline stage.  `limit_ns` is converted at 2 cycles per nanosecond, the most an SM of
// this part runs at, so the wait gives up no earlier than limit_ns and no later than about
// twice that at the lowest sustained clocks.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag,
                                          int site, uint64_t limit_ns, int kernel_id = 1) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  const long long limit_cycles = (long long)(limit_ns * 2ull);
  uint32_t spins = 0;
  while (true) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((++spins & 0x1Fu) == 0) {
      if (*abort_flag != 0) return false;
      if (clock64() - t0 > limit_cycles) {
        *abort_flag = 1;
        if (atomicCAS(&g_status[0], 0, ALTOB200_ETIMEOUT_DEVICE) == 0) {
          g_status[1] = kernel_id;  // 1 = a GEMM kernel, 9 = the wait self-test
          g_status[2] = (int)blockIdx.x;
          g_status[3] = site;
        }
        return false;
      }
    }
  }
}

// true in exactly one lane of a converged warp
__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "elect.sync _|p, 0xFFFFFFFF;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(pred));
  return pred != 0;
}
template <int N>
__device__ __forceinline__ void setmaxnreg_dec() {
  asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(N));
}
template <int N>
__device__ __forceinline__ void setmaxnreg_inc() {
  asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(N));
}

// Named-barrier rendezvous of `count` threads (whole warps) with an OR over a predicate: every
// participant learns whether any of them reports a failure.  A hardware barrier, not shared memory:
// it costs the MMA-issuing warp a few tens of cycles where an mbarrier wait between tcgen05.mma
// instructions costs ~150 (measured), during which the tensor pipe idles because tcgen05.mma does not
// run ahead of the issuing thread's other instructions.
__device__ __forceinline__ bool named_barrier_or(int id, int count, bool pred) {
  uint32_t r;
  asm volatile(
      "{\n\t.reg .pred p, q;\n\t"
      "setp.ne.b32 q, %3, 0;\n\t"
      "bar.red.or.pred p, %1, %2, q;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(r)
      : "r"(id), "r"(count), "r"((uint32_t)pred)
      : "memory");
  return r != 0;
}

__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* map, int32_t x, int32_t y,
                                            uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(smem_u32(smem_dst)), "l"(map), "r"(x), "r"(y), "r"(smem_u32(bar))
      : "memory");
}
__device__ __forceinline__ void bulk_load(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
      ::"r"(smem_u32(smem_dst)), "l"(gsrc), "r"(bytes), "r"(smem_u32(bar))
      : "memory");
}

__device__ __forceinline__ void tma_store_2d(const void* smem_src, const CUtensorMap* map, int32_t x, int32_t y) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
               ::"l"(map), "r"(smem_u32(smem_src)), "r"(x), "r"(y)
               : "memory");
}
__device__ __forceinline__ void tma_store_3d(const void* smem_src, const CUtensorMap* map, int32_t x, int32_t y,
                                             int32_t z) {
  asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%2, %3, %4}], [%1];"
               ::"l"(map), "r"(smem_u32(smem_src)), "r"(x), "r"(y), "r"(z)
               : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void bulk_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void st_shared_v4(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}

__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}
template <int KIND>
__device__ __forceinline__ void tc_mma(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                       uint32_t accumulate, uint32_t sfa, uint32_t sfb) {
  if (KIND == KIND_NVF4) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.block16 [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(sfa), "r"(sfb)
        : "memory");
  } else if (KIND == KIND_MXF4) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::mxf4.block_scale.block32 [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(sfa), "r"(sfb)
        : "memory");
  } else {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(sfa), "r"(sfb)
        : "memory");
  }
}
__device__ __forceinline__ void tc_ld32(uint32_t taddr, uint32_t* r) {
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
}
#define ALTOB200_R8(r, o) "=r"(r[o]), "=r"(r[o + 1]), "=r"(r[o + 2]), "=r"(r[o + 3]), "=r"(r[o + 4]), "=r"(r[o + 5]), \
                         "=r"(r[o + 6]), "=r"(r[o + 7])
__device__ __forceinline__ void tc_ld64(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x64.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, "
      "%32, %33, %34, %35, %36, %37, %38, %39, %40, %41, %42, %43, %44, %45, %46, %47, "
      "%48, %49, %50, %51, %52, %53, %54, %55, %56, %57, %58, %59, %60, %61, %62, %63}, [%64];"
      : ALTOB200_R8(r, 0), ALTOB200_R8(r, 8), ALTOB200_R8(r, 16), ALTOB200_R8(r, 24), ALTOB200_R8(r, 32),
        ALTOB200_R8(r, 40), ALTOB200_R8(r, 48), ALTOB200_R8(r, 56)
      : "r"(taddr)
      : "memory");
}
#undef ALTOB200_R8
__device__ __forceinline__ void tc_st4(uint32_t taddr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x4.b32 [%0], {%1, %2, %3, %4};" ::"r"(taddr), "r"(a), "r"(b), "r"(c),
               "r"(d)
               : "memory");
}
__device__ __forceinline__ void tc_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// High 32 bits of the operand descriptor (stride byte offset, version, swizzle); the low word
// holds the start address >> 4 (and the unused leading offset), so moving to another stage or
// 32-byte K slice is one 32-bit add for the single issuing thread.
constexpr uint32_t DESC_SW128_HI = (1024u >> 4) | (1u << 14) | (2u << 29);
__device__ __forceinline__ uint64_t desc_of(uint32_t hi, uint32_t lo) { return ((uint64_t)hi << 32) | lo; }

// Shared-memory matrix descriptor, K-major, 128-byte swizzle, 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t make_desc_sw128(uint32_t saddr) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr >> 4) & 0x3FFFu);      // start address
  d |= (uint64_t)1 << 16;                       // leading byte offset (unused for swizzled K-major)
  d |= (uint64_t)(1024 >> 4) << 32;             // stride byte offset
  d |= (uint64_t)1 << 46;                       // descriptor version (Blackwell)
  d |= (uint64_t)2 << 61;                       // SWIZZLE_128B
  return d;
}
// ---------------------------------------------------------------------------------------
// epilogue of one tile for one warp (its 32 accumulator rows), shared by both kernels
// ---------------------------------------------------------------------------------------
// The accumulator is drained in units of one 128-byte output row chunk (64 bf16 or 32 fp32 columns).
// The tensor-memory load of unit c+1 is in flight while unit c is scaled, converted, written to the
// 128-byte-swizzled staging buffer and handed to a TMA store; `release` (the arrival that gives the
// accumulator back to the MMA issuer) runs as soon as the last load has landed, before the last unit
// is converted.  NBUF 4 KB staging buffers per warp alternate; `store_it` carries the alternation
// across tiles.
template <int BN, int NBUF, class Release>
__device__ __forceinline__ void epilogue_tile(uint32_t t_acc, bool have_acc, float alpha, bool out_bf16,
                                              uint8_t* epi_warp, int lane, const CUtensorMap* tmap_d, int64_t row0,
                                              int64_t col_base, int batch, int64_t M, int64_t N, bool store_enabled,
                                              bool convert_enabled, uint32_t& store_it, Release release) {
  const uint32_t my_row = smem_u32(epi_warp) + (uint32_t)lane * 128u;  // this lane's 128-byte row (buffer 0)
  const uint32_t sw = (uint32_t)(lane & 7);                            // 16-byte chunk c -> c ^ (row & 7)
  auto stage_and_store = [&](int c, int cols_per_unit) {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    __syncwarp();
    const int64_t col0 = col_base + (int64_t)c * cols_per_unit;
    if (lane == 0) {
      if (row0 < M && col0 < N && store_enabled)
        tma_store_3d(epi_warp + (store_it % NBUF) * 4096u, tmap_d, (int32_t)col0, (int32_t)row0, batch);
      // a group is committed for every unit, empty when the unit lies outside the output: the
      // "all but the latest group have been read" wait before a buffer is refilled counts groups, so
      // a skipped unit must not let the store of the other buffer pass for the latest one
      bulk_commit();
    }
    ++store_it;
  };
  if (out_bf16) {
    // loads of 32 columns (half an output row chunk), two register buffers; a store every second load
    constexpr int NC = BN / 32;
    uint32_t rb[2][32];
    if (have_acc) tc_ld32(t_acc, rb[0]);
#pragma unroll
    for (int c = 0; c < NC; ++c) {
      uint32_t* r = rb[c & 1];
      const int h = c & 1;
      if (have_acc) {
        tc_wait_ld();
        if (c + 1 < NC) {
          tc_ld32(t_acc + (c + 1) * 32, rb[(c + 1) & 1]);
        } else {
          tc_fence_before();
          __syncwarp();
          if (lane == 0) release();
        }
      } else {
#pragma unroll
        for (int j = 0; j < 32; ++j) r[j] = 0u;
      }
      if (h == 0) {
        // the TMA store issued two chunks ago from this buffer must have finished reading it
        if (lane == 0) bulk_wait_read<NBUF - 1>();
        __syncwarp();
      }
      const uint32_t buf = my_row + (store_it % NBUF) * 4096u;
      if (convert_enabled)
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        uint32_t o[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          // one packed conversion per pair (round to nearest even, low half = first element)
          const __nv_bfloat162 p2 = __floats2bfloat162_rn(__fmul_rn(u2f(r[8 * j + 2 * q]), alpha),
                                                          __fmul_rn(u2f(r[8 * j + 2 * q + 1]), alpha));
          o[q] = *reinterpret_cast<const uint32_t*>(&p2);
        }
        st_shared_v4(buf + ((((uint32_t)(h * 4 + j)) ^ sw) << 4), o[0], o[1], o[2], o[3]);
      }
      if (h == 1) stage_and_store(c >> 1, 64);
    }
  } else {
    constexpr int NC = BN / 32;
    uint32_t rb[2][32];
    if (have_acc) tc_ld32(t_acc, rb[0]);
#pragma unroll
    for (int c = 0; c < NC; ++c) {
      uint32_t* r = rb[c & 1];
      if (have_acc) {
        tc_wait_ld();
        if (c + 1 < NC) {
          tc_ld32(t_acc + (c + 1) * 32, rb[(c + 1) & 1]);
        } else {
          tc_fence_before();
          __syncwarp();
          if (lane == 0) release();
        }
      } else {
#pragma unroll
        for (int j = 0; j < 32; ++j) r[j] = 0u;
      }
      if (lane == 0) bulk_wait_read<NBUF - 1>();
      __syncwarp();
      const uint32_t buf = my_row + (store_it % NBUF) * 4096u;
#pragma unroll
      for (int j = 0; j < 8; ++j)
        st_shared_v4(buf + ((((uint32_t)j) ^ sw) << 4), f2u(__fmul_rn(u2f(r[4 * j]), alpha)),
                     f2u(__fmul_rn(u2f(r[4 * j + 1]), alpha)), f2u(__fmul_rn(u2f(r[4 * j + 2]), alpha)),
                     f2u(__fmul_rn(u2f(r[4 * j + 3]), alpha)));
      stage_and_store(c, 32);
    }
  }
}

// ---------------------------------------------------------------------------------------
// kernel
// ---------------------------------------------------------------------------------------
template <int KIND, int BN>
struct Cfg {
  static constexpr int SF_TILES = Kind<KIND>::SF_TILES;
  static constexpr int NB = BN / 128;                        // 128-row blocks of B per tile
  static constexpr int A_BYTES = BM * STAGE_K_BYTES;         // 16 KiB
  static constexpr int B_BYTES = BN * STAGE_K_BYTES;
  static constexpr int SFA_BYTES = SF_TILES * 512;
  static constexpr int SFB_BYTES = NB * SF_TILES * 512;
  // rounded up so that every stage starts on a 1024-byte boundary (128-byte swizzle atom)
  static constexpr int STAGE_BYTES = (A_BYTES + B_BYTES + SFA_BYTES + SFB_BYTES + 1023) / 1024 * 1024;
  static constexpr int SF_COLS_A = SF_TILES * 4;             // tensor-memory columns per stage
  static constexpr int SF_COLS_B = SF_TILES * 4 * NB;
  static constexpr int ACC_STAGES = (BN <= 128) ? 2 : 1;
  static constexpr int STAGES = (BN == 256) ? 3 : 5;
  static constexpr int EPI_BYTES = 4 /*warps*/ * 2 /*buffers*/ * 4096;  // 32 rows x 128 bytes each
  static constexpr int TMEM_SF_BASE = ACC_STAGES * BN;
  static constexpr int TMEM_COLS_USED = TMEM_SF_BASE + STAGES * (SF_COLS_A + SF_COLS_B);
  static_assert(TMEM_COLS_USED <= 512, "tensor memory budget");
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + EPI_BYTES + 1024 /*align*/ + 256 /*barriers*/;
  static_assert(SMEM_BYTES <= 232448, "shared memory budget");
};

// What one output tile needs, identically derived by every role of the CTA.
struct TileInfo {
  int64_t mb, nb;      // tile coordinates
  int batch;           // z coordinate of the output (K-range mode), else 0
  int k_stages;        // stages of 128 bytes of K
  int last_mmas;       // MMAs issued in the last stage (a K range may end half-way through a stage)
  int64_t k_byte0;     // first byte of the K range in an operand row
  int64_t sf_tile0;    // first 512-byte scale tile of the K range
  int64_t b_row0;      // first row of the B tile in its tensor map
  const uint8_t* sfb;  // packed scales of B for this tile's expert
  bool skip;           // nothing to contract: the epilogue writes zeros
};

template <int KIND, int BN>
__device__ __forceinline__ TileInfo decode_tile(const GemmArgs& args, int64_t tile, int64_t tiles_m, int64_t tiles_n,
                                                int k_stages_dense) {
  TileInfo t;
  const int64_t per_batch = tiles_m * tiles_n;
  const int64_t e = args.k_offs != nullptr ? tile / per_batch : 0;
  const int64_t rem = tile - e * per_batch;
  // raster: groups of `group_m` row tiles, each group swept across all column tiles with the row
  // tile running fastest, so that the group's A rows stay in L2 while B streams once per group
  const int64_t per_group = (int64_t)args.group_m * tiles_n;
  const int64_t g = rem / per_group;
  const int64_t r2 = rem - g * per_group;
  const int64_t m0 = g * args.group_m;
  const int64_t gsz = (tiles_m - m0) < args.group_m ? (tiles_m - m0) : (int64_t)args.group_m;
  t.nb = r2 / gsz;
  t.mb = m0 + (r2 - t.nb * gsz);
  t.batch = (int)e;
  t.k_stages = k_stages_dense;
  t.last_mmas = 4;
  t.k_byte0 = 0;
  t.sf_tile0 = 0;
  t.b_row0 = t.nb * BN;
  t.sfb = args.sfb;
  t.skip = false;
  if (args.k_offs != nullptr) {
    constexpr int EPB = Kind<KIND>::ELEMS_PER_BYTE;
    const int64_t k0 = e > 0 ? __ldg(args.k_offs + e - 1) : 0;
    const int64_t k1 = __ldg(args.k_offs + e);
    const int64_t bytes = (k1 - k0) / EPB;
    t.skip = bytes <= 0;
    t.k_stages = (int)((bytes + STAGE_K_BYTES - 1) / STAGE_K_BYTES);
    const int64_t tail = bytes - (int64_t)(t.k_stages - 1) * STAGE_K_BYTES;
    t.last_mmas = (int)((tail + 31) / 32);
    t.k_byte0 = k0 / EPB;
    t.sf_tile0 = k0 / (Kind<KIND>::BLOCK * 4);
  } else if (args.num_experts > 0) {
    const int ex = __ldg(args.group_expert + t.mb);
    t.skip = ex < 0;
    if (!t.skip) {
      t.b_row0 += (int64_t)ex * args.N;
      t.sfb += (int64_t)ex * args.sfb_expert_stride;
    }
  }
  return t;
}

template <int KIND, int BN>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_blockscaled_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                        const __grid_constant__ CUtensorMap tmap_d, const GemmArgs args) {
  using C = Cfg<KIND, BN>;
  extern __shared__ uint8_t smem_raw[];
  // operand stages need 1024-byte alignment for the 128-byte swizzle
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* epi = smem + C::STAGES * C::STAGE_BYTES;  // 1024-byte aligned staging of the epilogue
  uint64_t* bars = reinterpret_cast<uint64_t*>(epi + C::EPI_BYTES);
  uint64_t* full_bar = bars;
  uint64_t* empty_bar = bars + C::STAGES;
  uint64_t* sf_full = bars + 2 * C::STAGES;
  uint64_t* acc_full = bars + 3 * C::STAGES;
  uint64_t* acc_empty = acc_full + C::ACC_STAGES;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + C::ACC_STAGES);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t tiles_m = (args.M + BM - 1) / BM;
  const int64_t tiles_n = (args.N + BN - 1) / BN;
  const int64_t n_tiles = tiles_m * tiles_n * (args.k_offs != nullptr ? args.num_batches : 1);
  const int k_stages = (int)((args.k_bytes + STAGE_K_BYTES - 1) / STAGE_K_BYTES);
  const int64_t n_row_blocks = (args.N + 127) / 128;

  if (threadIdx.x == 0) {
    for (int s = 0; s < C::STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
      mbar_init(&sf_full[s], 4);
    }
    for (int a = 0; a < C::ACC_STAGES; ++a) {
      mbar_init(&acc_full[a], 1);
      mbar_init(&acc_empty[a], 4);
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  // Scale staging areas start from zero so that a stage whose K range is ragged never
  // feeds uninitialised bytes (a NaN scale would poison the zero-filled codes).
  for (int s = 0; s < C::STAGES; ++s) {
    uint32_t* z = reinterpret_cast<uint32_t*>(smem + s * C::STAGE_BYTES + C::A_BYTES + C::B_BYTES);
    for (int i = threadIdx.x; i < (C::SFA_BYTES + C::SFB_BYTES) / 4; i += NUM_THREADS) z[i] = 0u;
  }
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], 512;" ::"r"(smem_u32(tmem_slot))
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // barriers, tensor memory and the zeroed scale staging are set up: from here on global memory is read
  // and written, which has to wait for the kernel in front of this one (programmatic dependent launch)
  grid_dependency_wait();

  if (warp == 0) {
    // ------------------------------ producer ------------------------------
    // Whole warp in the loop, one elected lane issues (uniform operands; see the CTA-pair kernel).
    const bool elected = elect_one();
    uint32_t it = 0;
    bool alive = true;
    for (int64_t tile = blockIdx.x; tile < n_tiles && alive; tile += gridDim.x) {
      const TileInfo ti = decode_tile<KIND, BN>(args, tile, tiles_m, tiles_n, k_stages);
      if (ti.skip) continue;  // nothing to load: the epilogue writes zeros
      const int64_t mb = ti.mb, nb = ti.nb;
      // 128-row blocks of B that exist (the last tile of a ragged N has fewer)
      int nb_valid = (int)(n_row_blocks - nb * C::NB);
      if (nb_valid > C::NB) nb_valid = C::NB;
      for (int ks = 0; ks < ti.k_stages; ++ks, ++it) {
        const int s = it % C::STAGES;
        alive = __all_sync(0xFFFFFFFFu,
                           mbar_wait(&empty_bar[s], ((it / C::STAGES) & 1) ^ 1, abort_flag, 1, args.wait_ns));
        if (!alive) break;
        uint8_t* st = smem + s * C::STAGE_BYTES;
        const int64_t cb0 = ti.sf_tile0 + (int64_t)ks * C::SF_TILES;
        int64_t sf_tiles = args.nct - cb0;
        if (sf_tiles > C::SF_TILES) sf_tiles = C::SF_TILES;
        const uint32_t sf_bytes = (uint32_t)sf_tiles * 512u;
        if (ALTOB200_DBG(args, 4) && it >= (uint32_t)C::STAGES) {
          if (elected) mbar_arrive(&full_bar[s]);
          continue;
        }
        const int32_t kx = (int32_t)(ti.k_byte0 + (int64_t)ks * STAGE_K_BYTES);
        if (elected) {
          mbar_expect_tx(&full_bar[s], C::A_BYTES + C::B_BYTES + sf_bytes * (1 + nb_valid));
          tma_load_2d(st, &tmap_a, kx, (int32_t)(mb * BM), &full_bar[s]);
          tma_load_2d(st + C::A_BYTES, &tmap_b, kx, (int32_t)ti.b_row0, &full_bar[s]);
          bulk_load(st + C::A_BYTES + C::B_BYTES, args.sfa + (mb * args.nct + cb0) * 512, sf_bytes, &full_bar[s]);
#pragma unroll
          for (int j = 0; j < C::NB; ++j)
            if (j < nb_valid)
              bulk_load(st + C::A_BYTES + C::B_BYTES + C::SFA_BYTES + j * C::SFA_BYTES,
                        ti.sfb + ((nb * C::NB + j) * args.nct + cb0) * 512, sf_bytes, &full_bar[s]);
        }
        __syncwarp();
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer ------------------------------
    // Whole warp, elected lane issues; the shared-memory barriers are waited on by warp 10, which
    // releases this warp once per stage through named barrier 1 + stage (see the CTA-pair kernel).
    const bool elected = elect_one();
    uint32_t it = 0, tile_it = 0;
    bool alive = true;
    const uint32_t smem_base = smem_u32(smem);
    for (int64_t tile = blockIdx.x; tile < n_tiles && alive; tile += gridDim.x) {
      const TileInfo ti = decode_tile<KIND, BN>(args, tile, tiles_m, tiles_n, k_stages);
      if (ti.skip) continue;
      const int acc = tile_it % C::ACC_STAGES;
      const uint32_t d_tmem = tmem_base + acc * BN;
      for (int ks = 0; ks < ti.k_stages; ++ks, ++it) {
        const int n_mma = (ks == ti.k_stages - 1) ? ti.last_mmas : 4;
        const int s = it % C::STAGES;
        if (named_barrier_or(1 + s, 64, false)) { alive = false; break; }
        tc_fence_after();
        const uint32_t st4 = (smem_base + (uint32_t)s * C::STAGE_BYTES) >> 4;  // stage address / 16
        const uint32_t sfa_t = tmem_base + C::TMEM_SF_BASE + s * (C::SF_COLS_A + C::SF_COLS_B);
        const uint32_t sfb_t = sfa_t + C::SF_COLS_A;
        const uint32_t a_lo = st4 | 0x10000u;
        const uint32_t b_lo = a_lo + (C::A_BYTES >> 4);
        if (elected) {
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            // MMA j covers bytes [32j, 32j+32) of the stage; its scale tile and byte offset
            // inside the tile depend on how many scales one MMA consumes.
            const int t = (KIND == KIND_NVF4) ? j : (KIND == KIND_MXF4 ? (j >> 1) : 0);
            if (j < n_mma)
              tc_mma<KIND>(d_tmem, desc_of(DESC_SW128_HI, a_lo + 2 * j), desc_of(DESC_SW128_HI, b_lo + 2 * j),
                           args.idesc[j], (ks | j) != 0 ? 1u : 0u, sfa_t + t * 4, sfb_t + t * 4 * C::NB);
          }
          tc_commit(&empty_bar[s]);
        }
        __syncwarp();
      }
      if (alive && elected) tc_commit(&acc_full[acc]);
      __syncwarp();
      ++tile_it;
    }
  } else if (warp == 10) {
    // ------------------------------ wait warp ------------------------------
    uint32_t it = 0, tile_it = 0;
    bool alive = true;
    for (int64_t tile = blockIdx.x; tile < n_tiles && alive; tile += gridDim.x) {
      const TileInfo ti = decode_tile<KIND, BN>(args, tile, tiles_m, tiles_n, k_stages);
      if (ti.skip) continue;
      const int acc = tile_it % C::ACC_STAGES;
      bool ok = mbar_wait(&acc_empty[acc], ((tile_it / C::ACC_STAGES) & 1) ^ 1, abort_flag, 2, args.wait_ns);
      for (int ks = 0; ks < ti.k_stages; ++ks, ++it) {
        const int s = it % C::STAGES;
        ok = ok && mbar_wait(&full_bar[s], (it / C::STAGES) & 1, abort_flag, 3, args.wait_ns);
        ok = ok && mbar_wait(&sf_full[s], (it / C::STAGES) & 1, abort_flag, 5, args.wait_ns);
        const bool failed = !__all_sync(0xFFFFFFFFu, ok);
        if (named_barrier_or(1 + s, 64, failed)) { alive = false; break; }
      }
      ++tile_it;
    }
  } else if (warp >= 6) {
    // ------------------------------ scale transfer (warps 6..9) ------------------------------
    // Tile t of A -> columns [4t, 4t+4) of the stage's A-scale area; tile t of B row block j ->
    // columns [4 NB t + 4 j, +4) of its B-scale area.  Lane l of every quarter holds scale row
    // l of each 512-byte tile (16 bytes = 4 columns), i.e. the 4x replicated layout the MMA reads.
    const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
    uint32_t it = 0;
    bool alive = true;
    for (int64_t tile = blockIdx.x; tile < n_tiles && alive; tile += gridDim.x) {
      const TileInfo ti = decode_tile<KIND, BN>(args, tile, tiles_m, tiles_n, k_stages);
      if (ti.skip) continue;
      for (int ks = 0; ks < ti.k_stages; ++ks, ++it) {
        const int s = it % C::STAGES;
        if (!mbar_wait(&full_bar[s], (it / C::STAGES) & 1, abort_flag, 6, args.wait_ns)) { alive = false; break; }
        const uint8_t* sf = smem + s * C::STAGE_BYTES + C::A_BYTES + C::B_BYTES + lane * 16;
        const uint32_t sfa_t = tmem_base + lane_base + C::TMEM_SF_BASE + s * (C::SF_COLS_A + C::SF_COLS_B);
        const uint32_t sfb_t = sfa_t + C::SF_COLS_A;
        if (!(ALTOB200_DBG(args, 1) && ks > 0)) {
#pragma unroll
          for (int t = 0; t < C::SF_TILES; ++t) {
            const uint4 a = *reinterpret_cast<const uint4*>(sf + t * 512);
            tc_st4(sfa_t + t * 4, a.x, a.y, a.z, a.w);
#pragma unroll
            for (int j = 0; j < C::NB; ++j) {
              const uint4 b = *reinterpret_cast<const uint4*>(sf + C::SFA_BYTES + j * C::SFA_BYTES + t * 512);
              tc_st4(sfb_t + t * 4 * C::NB + j * 4, b.x, b.y, b.z, b.w);
            }
          }
          tc_wait_st();
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&sf_full[s]);
      }
    }
  } else {
    // ------------------------------ epilogue ------------------------------
    const int quad = warp & 3;  // tensor-memory lane quarter this warp may read
    float alpha = 1.0f;
    if (args.alpha_a != nullptr) alpha = __fmul_rn(alpha, __ldg(args.alpha_a));
    if (args.alpha_b != nullptr) alpha = __fmul_rn(alpha, __ldg(args.alpha_b));
    uint32_t tile_it = 0, store_it = 0;
    for (int64_t tile = blockIdx.x; tile < n_tiles; tile += gridDim.x) {
      const TileInfo ti = decode_tile<KIND, BN>(args, tile, tiles_m, tiles_n, k_stages);
      const int64_t mb = ti.mb, nb = ti.nb;
      const int64_t row0 = mb * BM + quad * 32;
      const bool pad_group = ti.skip;
      const int acc = tile_it % C::ACC_STAGES;
      if (!pad_group) {
        if (!mbar_wait(&acc_full[acc], (tile_it / C::ACC_STAGES) & 1, abort_flag, 4, args.wait_ns)) break;
        tc_fence_after();
      }
      const uint32_t t_acc = tmem_base + ((uint32_t)(quad * 32) << 16) + acc * BN;
      if (ALTOB200_DBG(args, 8) && !pad_group) {
        // profiling only: hand the accumulator straight back (mainloop-only time, output unwritten)
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&acc_empty[acc]);
        ++tile_it;
        continue;
      }
      epilogue_tile<BN, 2>(t_acc, !pad_group, alpha, args.out_bf16 != 0, epi + (warp - 2) * 8192, lane, &tmap_d, row0,
                        nb * BN, ti.batch, args.M, args.N, !ALTOB200_DBG(args, 2), !ALTOB200_DBG(args, 32), store_it,
                        [&]() { mbar_arrive(&acc_empty[acc]); });
      if (!pad_group) ++tile_it;
    }
    if (lane == 0) bulk_wait_all();
  }

  // ------------------------------ teardown ------------------------------
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, 512;" ::"r"(tmem_base) : "memory");
  }
}

// ---------------------------------------------------------------------------------------
// CTA-pair kernel (tcgen05 cta_group::2)
// ---------------------------------------------------------------------------------------
// Two CTAs of a cluster share one 256 x 256 output tile: CTA r of the pair holds rows
// [128 r, 128 r + 128) of A, rows [128 r, 128 r + 128) of the B tile (half of its 256 N-columns) and,
// in its own tensor memory, the accumulator of its 128 output rows over all 256 columns.  One
// thread of the even CTA (the leader) issues every MMA for both; the instruction reads A and the
// B halves from both CTAs' shared memory at the same offsets.  Per 128x256x64 of work a CTA thus
// reads 8 KB of shared memory instead of 12 KB, and TMA writes 8 KB instead of 12 KB, which is what
// bounds the single-CTA kernel.  Scale factors: every CTA needs SFA of its own rows and SFB of all
// 256 columns in its own tensor memory; its scale-transfer warps put them there as before.
//
// Synchronisation (all mbarriers live in shared memory of the CTA named):
//   full[s]     leader   operand bytes of both CTAs (TMA from the peer completes on the leader's barrier)
//   sfs_full[s] each CTA its own scale bytes, for its scale-transfer warps
//   sf_full[s]  leader   8 arrivals: the 4 scale-transfer warps of each CTA
//   empty[s]    each CTA arrival by the leader's commit (sent to both CTAs)
//   acc_full    each CTA arrival by the leader's commit (sent to both CTAs)
//   acc_empty   leader   16 arrivals: the 8 epilogue warps of each CTA
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// shared::cluster address of the same shared-memory offset in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t mapa_u32(uint32_t local_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local_addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// Arrival without a cluster-scope release.  What the waiting side consumes after these arrivals
// is tensor memory, whose writes (tcgen05.st) and reads (tcgen05.ld) the arriving warp has already
// completed with tcgen05.wait and ordered with tcgen05.fence::before_thread_sync; a release fence at
// cluster scope in front of every arrival costs about a microsecond per stage (measured).
__device__ __forceinline__ void mbar_arrive_cluster_relaxed(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.relaxed.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// tiled load into this CTA's shared memory whose bytes complete on a barrier given as a
// shared::cluster address (the leader's)
__device__ __forceinline__ void tma_load_2d_pair(void* smem_dst, const CUtensorMap* map, int32_t x, int32_t y,
                                                 uint32_t bar_cluster_addr) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%2, %3}], [%4];"
      ::"r"(smem_u32(smem_dst)), "l"(map), "r"(x), "r"(y), "r"(bar_cluster_addr)
      : "memory");
}
// arrival on the barrier at this offset in both CTAs of the pair once all prior MMAs of this thread finish
__device__ __forceinline__ void tc_commit_pair(uint64_t* bar) {
  const uint16_t mask = 3;
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
      ::"r"(smem_u32(bar)), "h"(mask)
      : "memory");
}
template <int KIND>
__device__ __forceinline__ void tc_mma_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                            uint32_t accumulate, uint32_t sfa, uint32_t sfb) {
  if (KIND == KIND_NVF4) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::mxf4nvf4.block_scale.block16 [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(sfa), "r"(sfb)
        : "memory");
  } else if (KIND == KIND_MXF4) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::mxf4.block_scale.block32 [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(sfa), "r"(sfb)
        : "memory");
  } else {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(sfa), "r"(sfb)
        : "memory");
  }
}

// BN_ = 256: one accumulator stage (256 + scale columns fill the tensor memory).  BN_ = 192: two
// accumulator stages, so that a tile's epilogue runs under the next tile's mainloop; a 192-column
// tile starts either on a 128-row block of B scales or 64 rows into one, so its scale columns start
// at word 0 or word 2 of the two blocks kept in tensor memory.
template <int KIND, int BN_>
struct CfgPair {
  static constexpr int BN = BN_;                             // columns of the pair's tile
  static constexpr int ACC_STAGES = BN_ == 256 ? 1 : 2;
  static constexpr int SF_TILES = Kind<KIND>::SF_TILES;
  static constexpr int NB = 2;                               // 128-row blocks of B scales that a tile touches
  static constexpr int A_BYTES = BM * STAGE_K_BYTES;         // this CTA's 128 rows of A
  static constexpr int B_BYTES = (BN_ / 2) * STAGE_K_BYTES;  // this CTA's half of the B tile
  static constexpr int SFA_BYTES = SF_TILES * 512;
  static constexpr int SFB_BYTES = NB * SF_TILES * 512;
  static constexpr int STAGE_BYTES = (A_BYTES + B_BYTES + SFA_BYTES + SFB_BYTES + 1023) / 1024 * 1024;
  static constexpr int SF_COLS_A = SF_TILES * 4;
  static constexpr int SF_COLS_B = SF_TILES * 4 * NB;
  static constexpr int STAGES = 4;                           // (a fifth stage was measured: no gain)
  static constexpr int EPI_WARPS = 8;                        // two warps per tensor-memory lane quarter
  static constexpr int EPI_BUFS = 2;                         // 4 KB staging buffers per epilogue warp
  static constexpr int EPI_BYTES = EPI_WARPS * EPI_BUFS * 4096;
  // registers per thread after the warpgroups have re-divided the file: 2 x 128 x 56 + 2 x 128 x 200 = 65536
  static constexpr int REGS_SMALL = BN_ == 256 ? 56 : 72, REGS_EPI = BN_ == 256 ? 200 : 184;
  // setmaxnreg.inc takes only what setmaxnreg.dec released inside the CTA (launched at 128 per thread)
  static_assert(REGS_SMALL + REGS_EPI == 2 * 128, "setmaxnreg budget must balance");
  static constexpr int TMEM_SF_BASE = ACC_STAGES * BN;
  static constexpr int SF_COLS = SF_COLS_A + SF_COLS_B;
  // scale slots in tensor memory: one per operand stage if they fit, else as many as do (a slot is
  // then reused as soon as the MMAs of the stage that read it have completed)
  static constexpr int SF_SLOTS = (512 - TMEM_SF_BASE) / SF_COLS < STAGES ? (512 - TMEM_SF_BASE) / SF_COLS : STAGES;
  static_assert(SF_SLOTS >= 2, "tensor memory budget");
  static constexpr int TMEM_COLS_USED = TMEM_SF_BASE + SF_SLOTS * SF_COLS;
  static_assert(TMEM_COLS_USED <= 512, "tensor memory budget");
  static constexpr int HALF_COLS = BN / 2;                    // columns drained by one epilogue warp
  static constexpr int NUM_BARS = 4 * STAGES + 2 * ACC_STAGES;
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + EPI_BYTES + 1024 /*align*/ + 512 /*barriers*/;
  static_assert(NUM_BARS * 8 + 16 <= 512, "barrier area");
  static_assert(SMEM_BYTES <= 232448, "shared memory budget");
};

template <int KIND, bool OUT_BF16, int BN_>
__global__ void __launch_bounds__(NUM_THREADS_PAIR, 1)
gemm_blockscaled_pair_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                             const __grid_constant__ CUtensorMap tmap_d, const GemmArgs args) {
  using C = CfgPair<KIND, BN_>;
  constexpr int BN = C::BN;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* epi = smem + C::STAGES * C::STAGE_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(epi + C::EPI_BYTES);
  uint64_t* full_bar = bars;
  uint64_t* empty_bar = bars + C::STAGES;
  uint64_t* sfs_full = bars + 2 * C::STAGES;
  uint64_t* sf_full = bars + 3 * C::STAGES;
  uint64_t* acc_full = bars + 4 * C::STAGES;
  uint64_t* acc_empty = acc_full + C::ACC_STAGES;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + C::ACC_STAGES);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();      // 0 = leader
  const bool leader = rank == 0;
  const int64_t pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
  const int64_t tiles_m = (args.M + 2 * BM - 1) / (2 * BM);    // tiles of 256 rows
  const int64_t tiles_n = (args.N + BN - 1) / BN;
  const int64_t n_tiles = tiles_m * tiles_n * (args.k_offs != nullptr ? args.num_batches : 1);
  const int k_stages = (int)((args.k_bytes + STAGE_K_BYTES - 1) / STAGE_K_BYTES);
  const int64_t n_row_blocks = (args.N + 127) / 128;

  if (threadIdx.x == 0) {
    for (int s = 0; s < C::STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
      mbar_init(&sfs_full[s], 1);
      mbar_init(&sf_full[s], 8);
    }
    for (int a = 0; a < C::ACC_STAGES; ++a) {
      mbar_init(&acc_full[a], 1);
      mbar_init(&acc_empty[a], 2 * C::EPI_WARPS);
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  for (int s = 0; s < C::STAGES; ++s) {
    uint32_t* z = reinterpret_cast<uint32_t*>(smem + s * C::STAGE_BYTES + C::A_BYTES + C::B_BYTES);
    for (int i = threadIdx.x; i < (C::SFA_BYTES + C::SFB_BYTES) / 4; i += NUM_THREADS_PAIR) z[i] = 0u;
  }
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  if (warp == 1) {
    // both CTAs of the pair execute the paired allocation, with the same destination offset
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], 512;" ::"r"(smem_u32(tmem_slot))
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();   // the peer's barriers are initialised before anything can arrive on them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // barriers, tensor memory and the zeroed scale staging are set up: from here on global memory is read
  // and written, which has to wait for the kernel in front of this one (programmatic dependent launch)
  grid_dependency_wait();

  if (warp < 4) {
  setmaxnreg_dec<C::REGS_SMALL>();
  if (warp == 0) {
    // ------------------------------ producer (each CTA loads its own halves) ------------------------------
    // Whole warp in the loop, one elected lane issues: the copy instructions take uniform operands (see
    // the MMA issuer below).
    {
      const bool elected = elect_one();
      uint32_t it = 0;
      bool alive = true;
      for (int64_t tile = pair; tile < n_tiles && alive; tile += n_pairs) {
        const TileInfo ti = decode_tile<KIND, BN>(args, tile, tiles_m, tiles_n, k_stages);
        if (ti.skip) continue;
        const int64_t mb = ti.mb * 2 + rank;          // this CTA's 128-row block of A
        const int64_t sfb_blk0 = (ti.nb * BN) >> 7;   // first 128-row block of B scales under this tile
        int nb_valid = (int)(n_row_blocks - sfb_blk0);
        if (nb_valid > C::NB) nb_valid = C::NB;
        // a CTA whose rows of A lie past M has no scale row block to load; its rows are never stored
        const bool sfa_exists = mb * BM < args.M;
        const uint8_t* sfa_row = args.sfa + mb * args.nct * 512;
        for (int ks = 0; ks < ti.k_stages; ++ks, ++it) {
          const int s = it % C::STAGES;
          alive = __all_sync(0xFFFFFFFFu,
                             mbar_wait(&empty_bar[s], ((it / C::STAGES) & 1) ^ 1, abort_flag, 11, args.wait_ns));
          if (!alive) break;
          uint8_t* st = smem + s * C::STAGE_BYTES;
          const int64_t cb0 = ti.sf_tile0 + (int64_t)ks * C::SF_TILES;
          int64_t sf_tiles = args.nct - cb0;
          if (sf_tiles > C::SF_TILES) sf_tiles = C::SF_TILES;
          const uint32_t sf_bytes = (uint32_t)sf_tiles * 512u;
          const int32_t kx = (int32_t)(ti.k_byte0 + (int64_t)ks * STAGE_K_BYTES);
          if (ALTOB200_DBG(args, 4) && it >= (uint32_t)C::STAGES) {
            // profiling builds only: nothing is loaded once the ring has been filled
            if (elected) {
              if (leader) mbar_arrive(&full_bar[s]);
              mbar_arrive(&sfs_full[s]);
            }
            continue;
          }
          if (elected) {
            if (leader) mbar_expect_tx(&full_bar[s], 2 * (C::A_BYTES + C::B_BYTES));
            mbar_expect_tx(&sfs_full[s], sf_bytes * ((sfa_exists ? 1 : 0) + nb_valid));
            const uint32_t full_leader = mapa_u32(smem_u32(&full_bar[s]), 0);
            tma_load_2d_pair(st, &tmap_a, kx, (int32_t)(mb * BM), full_leader);
            tma_load_2d_pair(st + C::A_BYTES, &tmap_b, kx, (int32_t)(ti.b_row0 + rank * (BN / 2)), full_leader);
            if (sfa_exists) bulk_load(st + C::A_BYTES + C::B_BYTES, sfa_row + cb0 * 512, sf_bytes, &sfs_full[s]);
#pragma unroll
            for (int j = 0; j < C::NB; ++j)
              if (j < nb_valid)
                bulk_load(st + C::A_BYTES + C::B_BYTES + C::SFA_BYTES + j * C::SFA_BYTES,
                          ti.sfb + ((sfb_blk0 + j) * args.nct + cb0) * 512, sf_bytes, &sfs_full[s]);
          }
          __syncwarp();
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer (leader CTA only) ------------------------------
    // The whole warp runs the loop (so that descriptors and addresses are warp-uniform values), one
    // elected lane issues.  It never waits on a shared-memory barrier itself: warp 2 does and meets it
    // at named barrier 1 + stage.  Between two tcgen05.mma nothing but their operand arithmetic runs.
    if (leader) {
      const bool elected = elect_one();
      uint32_t it = 0, tile_it = 0;
      bool alive = true;
      const uint32_t smem_base = smem_u32(smem);
#ifdef ALTOB200_GEMM_PROFILE
      long long pk_mma = 0, pk_bar = 0, pk_n = 0;
      const long long pk_t0 = clock64();
#endif
      for (int64_t tile = pair; tile < n_tiles && alive; tile += n_pairs) {
        const TileInfo ti = decode_tile<KIND, BN>(args, tile, tiles_m, tiles_n, k_stages);
        if (ti.skip) continue;
        const uint32_t acc = tile_it % C::ACC_STAGES;
        const uint32_t d_tmem = tmem_base + acc * BN;
        // scale columns of B start at word 0 of the first block, or 64 rows (2 words) into it
        const uint32_t sfb_off = (uint32_t)((ti.nb * BN) & 127) >> 5;
        for (int ks = 0; ks < ti.k_stages; ++ks, ++it) {
          const int n_mma = (ks == ti.k_stages - 1) ? ti.last_mmas : 4;
          const int s = it % C::STAGES;
          // operands and scales of the stage are in place (and, at ks == 0, the accumulator is free)
#ifdef ALTOB200_GEMM_PROFILE
          const long long pk_a = clock64();
#endif
          if (named_barrier_or(1 + s, 64, false)) { alive = false; break; }
          if (!ALTOB200_DBG(args, 2048)) tc_fence_after();
          const uint32_t st4 = (smem_base + (uint32_t)s * C::STAGE_BYTES) >> 4;
          const uint32_t sfa_t = tmem_base + C::TMEM_SF_BASE + (it % C::SF_SLOTS) * C::SF_COLS;
          const uint32_t sfb_t = sfa_t + C::SF_COLS_A + sfb_off;
          const uint32_t a_lo = st4 | 0x10000u;
          const uint32_t b_lo = a_lo + (C::A_BYTES >> 4);
#ifdef ALTOB200_GEMM_PROFILE
          const long long pk_b = clock64();
          pk_bar += pk_b - pk_a;
#endif
          if (elected) {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const int t = (KIND == KIND_NVF4) ? j : (KIND == KIND_MXF4 ? (j >> 1) : 0);
              if (j < n_mma)
                tc_mma_pair<KIND>(d_tmem, desc_of(DESC_SW128_HI, a_lo + 2 * j), desc_of(DESC_SW128_HI, b_lo + 2 * j),
                                  args.idesc[j], (ks | j) != 0 ? 1u : 0u, sfa_t + t * 4, sfb_t + t * 4 * C::NB);
            }
            tc_commit_pair(&empty_bar[s]);
          }
          __syncwarp();
#ifdef ALTOB200_GEMM_PROFILE
          pk_mma += clock64() - pk_b;
          pk_n += 1;
#endif
        }
        if (alive && elected) tc_commit_pair(&acc_full[acc]);
        __syncwarp();
        ++tile_it;
      }
#ifdef ALTOB200_GEMM_PROFILE
      if (blockIdx.x == 0 && lane == 0 && (args.debug & 16384))
        printf("pair MMA warp: %lld stages, per stage: total %lld, barrier+fence+address %lld, issue of 4 MMAs + commit %lld cycles\n", pk_n,
               (clock64() - pk_t0) / (pk_n > 0 ? pk_n : 1), pk_bar / (pk_n > 0 ? pk_n : 1), pk_mma / (pk_n > 0 ? pk_n : 1));
#endif
    }
  } else if (warp == 2) {
    // ------------------------------ wait warp (leader CTA only) ------------------------------
    // Waits on the shared-memory barriers on behalf of the MMA issuer and releases it per stage.
    if (leader) {
      uint32_t it = 0, tile_it = 0;
      bool alive = true;
      for (int64_t tile = pair; tile < n_tiles && alive; tile += n_pairs) {
        const TileInfo ti = decode_tile<KIND, BN>(args, tile, tiles_m, tiles_n, k_stages);
        if (ti.skip) continue;
        bool ok = mbar_wait(&acc_empty[tile_it % C::ACC_STAGES], ((tile_it / C::ACC_STAGES) & 1) ^ 1, abort_flag, 12,
                            args.wait_ns);
        for (int ks = 0; ks < ti.k_stages; ++ks, ++it) {
          const int s = it % C::STAGES;
          ok = ok && mbar_wait(&full_bar[s], (it / C::STAGES) & 1, abort_flag, 13, args.wait_ns);
          ok = ok && mbar_wait(&sf_full[s], (it / C::STAGES) & 1, abort_flag, 15, args.wait_ns);
          const bool failed = !__all_sync(0xFFFFFFFFu, ok);
          if (named_barrier_or(1 + s, 64, failed)) { alive = false; break; }
        }
        ++tile_it;
      }
    }
  }  // warp 3 idles: it completes warpgroup 0
  } else if (warp < 8) {
    // ------------------------------ scale transfer (each CTA into its own tensor memory) ------------------------------
    setmaxnreg_dec<C::REGS_SMALL>();
    const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
    uint32_t it = 0;
    bool alive = true;
    for (int64_t tile = pair; tile < n_tiles && alive; tile += n_pairs) {
      const TileInfo ti = decode_tile<KIND, BN>(args, tile, tiles_m, tiles_n, k_stages);
      if (ti.skip) continue;
      for (int ks = 0; ks < ti.k_stages; ++ks, ++it) {
        const int s = it % C::STAGES;
        if (!mbar_wait(&sfs_full[s], (it / C::STAGES) & 1, abort_flag, 16, args.wait_ns)) { alive = false; break; }
        if (C::SF_SLOTS < C::STAGES && it >= (uint32_t)C::SF_SLOTS) {
          // fewer scale slots than operand stages: the slot is free once the MMAs that read it have
          // completed, which is what frees the operand stage of that earlier step as well
          const uint32_t prev = it - C::SF_SLOTS;
          if (!mbar_wait(&empty_bar[prev % C::STAGES], (prev / C::STAGES) & 1, abort_flag, 17, args.wait_ns)) {
            alive = false;
            break;
          }
          tc_fence_after();
        }
        const uint8_t* sf = smem + s * C::STAGE_BYTES + C::A_BYTES + C::B_BYTES + lane * 16;
        const uint32_t sfa_t = tmem_base + lane_base + C::TMEM_SF_BASE + (it % C::SF_SLOTS) * C::SF_COLS;
        const uint32_t sfb_t = sfa_t + C::SF_COLS_A;
#pragma unroll
        for (int t = 0; t < C::SF_TILES; ++t) {
          const uint4 a = *reinterpret_cast<const uint4*>(sf + t * 512);
          tc_st4(sfa_t + t * 4, a.x, a.y, a.z, a.w);
#pragma unroll
          for (int j = 0; j < C::NB; ++j) {
            const uint4 b = *reinterpret_cast<const uint4*>(sf + C::SFA_BYTES + j * C::SFA_BYTES + t * 512);
            tc_st4(sfb_t + t * 4 * C::NB + j * 4, b.x, b.y, b.z, b.w);
          }
        }
        tc_wait_st();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) {
          if (leader) mbar_arrive(&sf_full[s]);
          else mbar_arrive_cluster_relaxed(mapa_u32(smem_u32(&sf_full[s]), 0));
        }
      }
    }
  } else {
    // ------------------------------ epilogue (each CTA stores its own 128 rows) ------------------------------
    // Warps 8-11 drain the first half of the accumulator's columns, warps 12-15 the second half; a
    // warp may read the tensor-memory lane quarter (warp index mod 4).  A warp first pulls its 32 rows
    // x BN/2 columns into registers (all loads in flight, one wait) and hands the accumulator back;
    // scaling, conversion, staging and the TMA stores then run under the next mainloop (with two
    // accumulator stages the tensor-memory read itself is under the next tile's mainloop as well).
    setmaxnreg_inc<C::REGS_EPI>();
    constexpr int HC = C::HALF_COLS;
    // one staged unit = 32 rows x UNIT_BYTES: 128-byte rows (128-byte swizzle) when they divide the
    // half tile, else 64-byte rows (64-byte swizzle; the output tensor map is built to match)
    constexpr int ESZ = OUT_BF16 ? 2 : 4;
    constexpr int UNIT_BYTES = (HC * ESZ) % 128 == 0 ? 128 : 64;
    constexpr int UNIT_COLS = UNIT_BYTES / ESZ;
    constexpr int N_UNITS = HC / UNIT_COLS;
    constexpr int CHUNKS = UNIT_BYTES / 16;       // 16-byte chunks per staged row
    constexpr int CHUNK_COLS = 16 / ESZ;
    const int quad = warp & 3;
    const int half = warp >= 12 ? 1 : 0;
    const int epi_idx = warp - 8;
    uint8_t* epi_warp = epi + epi_idx * (C::EPI_BUFS * 4096);
    float alpha = 1.0f;
    if (args.alpha_a != nullptr) alpha = __fmul_rn(alpha, __ldg(args.alpha_a));
    if (args.alpha_b != nullptr) alpha = __fmul_rn(alpha, __ldg(args.alpha_b));
    const uint32_t my_row = smem_u32(epi_warp) + (uint32_t)lane * (uint32_t)UNIT_BYTES;
    const uint32_t sw = UNIT_BYTES == 128 ? (uint32_t)(lane & 7) : (uint32_t)((lane >> 1) & 3);
    uint32_t tile_it = 0, store_it = 0;
    for (int64_t tile = pair; tile < n_tiles; tile += n_pairs) {
      const TileInfo ti = decode_tile<KIND, BN>(args, tile, tiles_m, tiles_n, k_stages);
      const int64_t row0 = (ti.mb * 2 + rank) * BM + quad * 32;
      const int64_t col_base = ti.nb * BN + half * HC;
      uint32_t r[HC];
      if (!ti.skip) {
        const uint32_t acc = tile_it % C::ACC_STAGES;
        if (!mbar_wait(&acc_full[acc], (tile_it / C::ACC_STAGES) & 1, abort_flag, 14, args.wait_ns)) break;
        tc_fence_after();
        if (!ALTOB200_DBG(args, 8)) {
          const uint32_t t_acc = tmem_base + ((uint32_t)(quad * 32) << 16) + acc * BN + half * HC;
#pragma unroll
          for (int c = 0; c < HC / 32; ++c) tc_ld32(t_acc + c * 32, r + c * 32);
          tc_wait_ld();
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) {
          if (leader) mbar_arrive(&acc_empty[acc]);
          else mbar_arrive_cluster_relaxed(mapa_u32(smem_u32(&acc_empty[acc]), 0));
        }
        ++tile_it;
        if (ALTOB200_DBG(args, 8)) continue;
      } else {
#pragma unroll
        for (int q = 0; q < HC; ++q) r[q] = 0u;
      }
#pragma unroll
      for (int u = 0; u < N_UNITS; ++u) {
        if (lane == 0) bulk_wait_read<C::EPI_BUFS - 1>();  // the store that last used this buffer has read it
        __syncwarp();
        const uint32_t buf = my_row + (store_it % C::EPI_BUFS) * 4096u;
#pragma unroll
        for (int q = 0; q < CHUNKS; ++q) {
          uint32_t o[4];
          if (OUT_BF16) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const __nv_bfloat162 p2 =
                  __floats2bfloat162_rn(__fmul_rn(u2f(r[u * UNIT_COLS + q * CHUNK_COLS + 2 * e]), alpha),
                                        __fmul_rn(u2f(r[u * UNIT_COLS + q * CHUNK_COLS + 2 * e + 1]), alpha));
              o[e] = *reinterpret_cast<const uint32_t*>(&p2);
            }
          } else {
#pragma unroll
            for (int e = 0; e < 4; ++e) o[e] = f2u(__fmul_rn(u2f(r[u * UNIT_COLS + q * CHUNK_COLS + e]), alpha));
          }
          st_shared_v4(buf + ((((uint32_t)q) ^ sw) << 4), o[0], o[1], o[2], o[3]);
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncwarp();
        const int64_t col0 = col_base + (int64_t)u * UNIT_COLS;
        if (lane == 0) {
          if (row0 < args.M && col0 < args.N && !ALTOB200_DBG(args, 2))
            tma_store_3d(epi_warp + (store_it % C::EPI_BUFS) * 4096u, &tmap_d, (int32_t)col0, (int32_t)row0, ti.batch);
          bulk_commit();  // one group per unit, empty or not: the wait above counts groups
        }
        ++store_it;
      }
    }
    if (lane == 0) bulk_wait_all();
  }

  // ------------------------------ teardown ------------------------------
  // Neither CTA may leave while its peer can still arrive on its barriers or read its shared memory.
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, 512;" ::"r"(tmem_base) : "memory");
  }
}

#include "gemm_macro.cuh"

// ---------------------------------------------------------------------------------------
// self-test of the bounded wait: one CTA, one thread waits on an mbarrier nobody arrives on
// ---------------------------------------------------------------------------------------
__global__ void __launch_bounds__(32, 1) wait_selftest_kernel(uint64_t limit_ns) {
  __shared__ uint64_t bar;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);
    abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  // phase 0 never completes (no arrival is ever made): the wait runs into its limit, records
  // {kernel 9, block, site 99} in the status word and returns false; the kernel then ends normally
  if (threadIdx.x == 0) (void)mbar_wait(&bar, 0, &abort_flag, 99, limit_ns, 9);
  __syncthreads();
}

// ---------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------
static std::atomic<uint64_t> g_wait_limit_ns{WAIT_LIMIT_NS};
static uint64_t wait_limit_ns() { return g_wait_limit_ns.load(std::memory_order_relaxed); }

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (fn == nullptr) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

// 3D tensor map of the output [batches, M, N] (bf16 or fp32): box of 1 x 32 rows x 128 bytes with
// the 128-byte swizzle, or x 64 bytes with the 64-byte swizzle (epilogues whose column share is not
// a multiple of 128 bytes).  The batch coordinate keeps a ragged tile of one batch entry out of the next.
static int make_tmap_out(CUtensorMap* m, void* base, int64_t batches, int64_t M, int64_t N, int64_t ldd, bool bf16,
                         int row_bytes = 128) {
  EncodeTiledFn fn = get_encode_fn();
  if (fn == nullptr) return ALTOB200_ECUDA;
  const int esz = bf16 ? 2 : 4;
  cuuint64_t dims[3] = {(cuuint64_t)N, (cuuint64_t)M, (cuuint64_t)batches};
  cuuint64_t strides[2] = {(cuuint64_t)(ldd * esz), (cuuint64_t)(M * ldd * esz)};
  cuuint32_t box[3] = {(cuuint32_t)(row_bytes / esz), 32u, 1u};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(m, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, base, dims, strides,
                  box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  row_bytes == 128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B,
                  CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? ALTOB200_OK : ALTOB200_ECUDA;
}

// 2D uint8 tensor map over [rows, row_bytes] with a box of [box_rows, 128 bytes].
static int make_tmap(CUtensorMap* m, const void* base, int64_t rows, int64_t row_bytes, int box_rows) {
  EncodeTiledFn fn = get_encode_fn();
  if (fn == nullptr) return ALTOB200_ECUDA;
  cuuint64_t dims[2] = {(cuuint64_t)row_bytes, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)row_bytes};
  cuuint32_t box[2] = {(cuuint32_t)STAGE_K_BYTES, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? ALTOB200_OK : ALTOB200_ECUDA;
}

// Instruction descriptor of a block-scaled MMA (bit layout: b_sf_id [4,6), a_format [7,10),
// b_format [10,13), n/8 [17,23), scale format [23], m/16 [24,29), a_sf_id [29,31)).
static uint32_t make_idesc(int kind, int fmt_a, int fmt_b, int m, int n, int sf_id) {
  uint32_t af, bf, sfmt;
  if (kind == KIND_MXF8) {
    af = fmt_a == ALTOB200_FMT_MXFP8_E5M2 ? 1u : 0u;
    bf = fmt_b == ALTOB200_FMT_MXFP8_E5M2 ? 1u : 0u;
    sfmt = 1u;
  } else {
    af = bf = 1u;  // E2M1
    sfmt = kind == KIND_NVF4 ? 0u : 1u;
  }
  uint32_t d = 0;
  d |= (uint32_t)sf_id << 4;
  d |= af << 7;
  d |= bf << 10;
  d |= (uint32_t)(n >> 3) << 17;
  d |= sfmt << 23;
  d |= (uint32_t)(m >> 4) << 24;
  d |= (uint32_t)sf_id << 29;
  return d;
}

// Per-device launch state.  A process may drive several GPUs (one context each): the dynamic
// shared-memory attribute of a kernel, the SM count and the number of resident clusters belong to
// the device that is current at the launch, so they are kept per device ordinal.  Entries are
// written with relaxed atomics: concurrent first calls compute the same values.
constexpr int MAX_DEVICES = 64;
static int current_device() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= MAX_DEVICES) return -1;
  return dev;
}
static int sm_count_gemm() {
  static std::atomic<int> n[MAX_DEVICES];
  const int dev = current_device();
  if (dev < 0) return 148;
  int v = n[dev].load(std::memory_order_relaxed);
  if (v == 0) {
    if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || v <= 0) v = 148;
    n[dev].store(v, std::memory_order_relaxed);
  }
  return v;
}
// Sets the dynamic shared-memory limit of `kernel` once per device.
template <class K>
static int ensure_smem_attr(K kernel, int bytes, std::atomic<int>* done /*[MAX_DEVICES]*/) {
  const int dev = current_device();
  if (dev >= 0 && done[dev].load(std::memory_order_relaxed) != 0) return ALTOB200_OK;
  ALTOB200_CUDA_CHECK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes));
  if (dev >= 0) done[dev].store(1, std::memory_order_relaxed);
  return ALTOB200_OK;
}

template <int KIND, int BN>
static int launch_gemm(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& td, const GemmArgs& args,
                       cudaStream_t st) {
  using C = Cfg<KIND, BN>;
  static std::atomic<int> attr_set[MAX_DEVICES];
  const int rc = ensure_smem_attr(gemm_blockscaled_kernel<KIND, BN>, C::SMEM_BYTES, attr_set);
  if (rc != ALTOB200_OK) return rc;
  const int64_t tiles = ceil_div(args.M, BM) * ceil_div(args.N, BN) * (args.k_offs != nullptr ? args.num_batches : 1);
  int64_t grid = sm_count_gemm();
  if (grid > tiles) grid = tiles;
  const cudaError_t e = launch_after(gemm_blockscaled_kernel<KIND, BN>, dim3((unsigned)grid), dim3(NUM_THREADS), C::SMEM_BYTES, st,
                                     ta, tb, td, args);
  return e == cudaSuccess ? ALTOB200_OK : ALTOB200_ECUDA;
}

// CTA-pair kernel: clusters of two CTAs, as many clusters as the device can hold at once.
template <int KIND, bool OUT_BF16, int BN_>
static int launch_gemm_pair(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& td, const GemmArgs& args,
                            cudaStream_t st) {
  using C = CfgPair<KIND, BN_>;
  static std::atomic<int> clusters_of[MAX_DEVICES];  // 0 = not asked yet, < 0 = the device cannot run the pair kernel
  const int dev = current_device();
  int max_clusters = dev >= 0 ? clusters_of[dev].load(std::memory_order_relaxed) : 0;
  cudaLaunchConfig_t cfg = {};
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;   // see launch_after()
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.blockDim = dim3(NUM_THREADS_PAIR, 1, 1);
  cfg.dynamicSmemBytes = C::SMEM_BYTES;
  cfg.stream = st;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_enabled() ? 2 : 1;
  if (max_clusters == 0) {
    ALTOB200_CUDA_CHECK(cudaFuncSetAttribute(gemm_blockscaled_pair_kernel<KIND, OUT_BF16, BN_>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES));
    cfg.gridDim = dim3(2 * (unsigned)sm_count_gemm(), 1, 1);
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, gemm_blockscaled_pair_kernel<KIND, OUT_BF16, BN_>, &cfg) != cudaSuccess || n <= 0) {
      (void)cudaGetLastError();
      max_clusters = -1;
    } else {
      max_clusters = n;
    }
    if (dev >= 0) clusters_of[dev].store(max_clusters, std::memory_order_relaxed);
  }
  if (max_clusters < 0) return ALTOB200_EUNSUPPORTED;
  const int64_t tiles =
      ceil_div(args.M, 2 * BM) * ceil_div(args.N, C::BN) * (args.k_offs != nullptr ? args.num_batches : 1);
  int64_t clusters = max_clusters;
  if (clusters > tiles) clusters = tiles;
  cfg.gridDim = dim3((unsigned)(2 * clusters), 1, 1);
  cudaError_t e = cudaLaunchKernelEx(&cfg, gemm_blockscaled_pair_kernel<KIND, OUT_BF16, BN_>, ta, tb, td, args);
  return e == cudaSuccess ? ALTOB200_OK : ALTOB200_ECUDA;
}

// Columns of the CTA-pair tile: 192 (two accumulator stages) or 256 (one); ALTOB200_PAIR_BN overrides.
static int pair_tile_n() {
  static int v = -1;
  if (v < 0) {
    const char* e = getenv("ALTOB200_PAIR_BN");
    const int n = e ? atoi(e) : 0;
    v = (n == 192 || n == 256) ? n : 256;
  }
  return v;
}

static int gemm_common(int32_t format_a, int32_t format_b, int64_t M, int64_t N, int64_t K, int32_t num_experts,
                       const void* a_codes, const void* a_scales, const void* b_codes, const void* b_scales,
                       const int32_t* group_expert, const float* alpha_a, const float* alpha_b,
                       int32_t out_dtype, void* d, int64_t ldd, void* stream, const int32_t* k_offs = nullptr,
                       int32_t num_batches = 1) {
  if (a_codes == nullptr || b_codes == nullptr || a_scales == nullptr || b_scales == nullptr || d == nullptr)
    return ALTOB200_EINVAL_SHAPE;
  int kind;
  if (format_a == ALTOB200_FMT_NVFP4 && format_b == ALTOB200_FMT_NVFP4) kind = KIND_NVF4;
  else if (format_a == ALTOB200_FMT_MXFP4 && format_b == ALTOB200_FMT_MXFP4) kind = KIND_MXF4;
  else if ((format_a == ALTOB200_FMT_MXFP8_E4M3 || format_a == ALTOB200_FMT_MXFP8_E5M2) &&
           (format_b == ALTOB200_FMT_MXFP8_E4M3 || format_b == ALTOB200_FMT_MXFP8_E5M2)) kind = KIND_MXF8;
  else return ALTOB200_EUNSUPPORTED;
  const int epb = kind == KIND_MXF8 ? 1 : 2;
  const int block = kind == KIND_NVF4 ? 16 : 32;
  if (M <= 0 || N <= 0 || K <= 0 || K % 32 != 0 || ldd < N) return ALTOB200_EINVAL_SHAPE;
  if (num_experts > 0 && group_expert == nullptr) return ALTOB200_EINVAL_SHAPE;
  const int64_t k_bytes = K / epb;
  if (k_bytes % 16 != 0) return ALTOB200_EINVAL_SHAPE;
  const int osz = out_dtype == ALTOB200_DT_BF16 ? 2 : 4;
  if ((reinterpret_cast<uintptr_t>(a_codes) & 15) || (reinterpret_cast<uintptr_t>(b_codes) & 15) ||
      (reinterpret_cast<uintptr_t>(a_scales) & 15) || (reinterpret_cast<uintptr_t>(b_scales) & 15) ||
      (reinterpret_cast<uintptr_t>(d) & 15) || (ldd * osz) % 16 != 0)
    return ALTOB200_EINVAL_ALIGN;
  if (M >= (1ll << 31) || N * (num_experts > 0 ? num_experts : 1) >= (1ll << 31) || k_bytes >= (1ll << 31))
    return ALTOB200_ELIMIT;

  int BN = N <= 128 ? 128 : 256;
  // The CTA-pair kernel serves dense and K-range problems; rows grouped by expert in runs of 128
  // could put two experts' rows into one 256-row pair tile, so that mode stays on the single-CTA
  // kernel.  ALTOB200_GEMM_PAIR=0 forces the single-CTA kernel everywhere.
  static int pair_env = -1;
  if (pair_env < 0) {
    const char* e = getenv("ALTOB200_GEMM_PAIR");
    pair_env = e ? atoi(e) : 1;
  }
  const bool use_pair = pair_env != 0 && num_experts == 0 && N > 128 && M > 128;
  if (use_pair && pair_tile_n() == 192) BN = 192;
  const int64_t b_rows = N * (num_experts > 0 ? num_experts : 1);
  CUtensorMap ta, tb;
  int rc = make_tmap(&ta, a_codes, M, k_bytes, BM);
  if (rc != ALTOB200_OK) return rc;
  rc = make_tmap(&tb, b_codes, b_rows, k_bytes, use_pair ? BN / 2 : BN);
  if (rc != ALTOB200_OK) return rc;
  CUtensorMap td;
  rc = make_tmap_out(&td, d, k_offs != nullptr ? num_batches : 1, M, N, ldd, out_dtype == ALTOB200_DT_BF16,
                     (use_pair && BN == 192 && out_dtype == ALTOB200_DT_BF16) ? 64 : 128);
  if (rc != ALTOB200_OK) return rc;

  GemmArgs g;
  g.M = M; g.N = N; g.K = K; g.k_bytes = k_bytes;
  g.sfa = (const uint8_t*)a_scales; g.sfb = (const uint8_t*)b_scales;
  g.nct = ceil_div(K / block, 4);
  g.alpha_a = alpha_a; g.alpha_b = alpha_b;
  g.d = d; g.ldd = ldd; g.out_bf16 = out_dtype == ALTOB200_DT_BF16;
  g.num_experts = num_experts; g.group_expert = group_expert;
  g.sfb_expert_stride = (int64_t)altob200_packed_scale_bytes(N, K / block);
  g.k_offs = k_offs; g.num_batches = num_batches;
  {
    // Row tiles per raster group: walking the whole M axis first re-reads A once per wave; a handful of
    // row tiles per group keeps a group's A rows in L2 while B streams once per group.
    const int64_t tiles_m = ceil_div(M, use_pair ? 2 * BM : BM);
    int64_t gm = use_pair ? 4 : 8;
    static int gm_env = -1;
    if (gm_env < 0) {
      const char* e = getenv("ALTOB200_GEMM_GROUP_M");
      gm_env = e ? atoi(e) : 0;
    }
    if (gm_env > 0) gm = gm_env;
    if (gm < 1) gm = 1;
    if (gm > tiles_m) gm = tiles_m;
    // even out the groups: same number of groups, near-equal sizes
    const int64_t n_groups = ceil_div(tiles_m, gm);
    gm = ceil_div(tiles_m, n_groups);
    g.group_m = (int)gm;
  }
  g.wait_ns = wait_limit_ns();
  for (int j = 0; j < 4; ++j) {
    const int sf_id = kind == KIND_NVF4 ? 0 : (kind == KIND_MXF4 ? (j & 1) * 2 : j);
    g.idesc[j] = make_idesc(kind, format_a, format_b, use_pair ? 2 * BM : BM, BN, sf_id);
  }
#ifdef ALTOB200_GEMM_PROFILE
  {
    const char* e = getenv("ALTOB200_GEMM_DEBUG");  // read at every call: probe scripts change it between calls
    g.debug = e ? atoi(e) : 0;
  }
#endif
  cudaStream_t st = (cudaStream_t)stream;
  if (use_pair) {
    const bool obf = g.out_bf16 != 0;
#define LAUNCH_PAIR(KD)                                                                                        \
  return BN == 192 ? (obf ? launch_gemm_pair<KD, true, 192>(ta, tb, td, g, st)                                \
                          : launch_gemm_pair<KD, false, 192>(ta, tb, td, g, st))                              \
                   : (obf ? launch_gemm_pair<KD, true, 256>(ta, tb, td, g, st)                                \
                          : launch_gemm_pair<KD, false, 256>(ta, tb, td, g, st))
    switch (kind) {
      case KIND_NVF4: LAUNCH_PAIR(KIND_NVF4);
      case KIND_MXF4: LAUNCH_PAIR(KIND_MXF4);
      default: LAUNCH_PAIR(KIND_MXF8);
    }
#undef LAUNCH_PAIR
  }
#define LAUNCH(KD)                                                    \
  return BN == 128 ? launch_gemm<KD, 128>(ta, tb, td, g, st) : launch_gemm<KD, 256>(ta, tb, td, g, st)
  switch (kind) {
    case KIND_NVF4: LAUNCH(KIND_NVF4);
    case KIND_MXF4: LAUNCH(KIND_MXF4);
    default: LAUNCH(KIND_MXF8);
  }
#undef LAUNCH
}

static int launch_gemm_macro(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& td,
                             const MacroGemmArgs& margs, cudaStream_t st) {
  using C = CfgMacro;
  static std::atomic<int> attr_set[MAX_DEVICES];
  const int rc = ensure_smem_attr(gemm_macro_kernel, C::SMEM_BYTES, attr_set);
  if (rc != ALTOB200_OK) return rc;
  const GemmArgs& a = margs.g;
  const int64_t tiles = ceil_div(a.M, BM) * ceil_div(a.N, C::BN) * (a.k_offs != nullptr ? a.num_batches : 1);
  int64_t grid = sm_count_gemm();
  if (grid > tiles) grid = tiles;
  (void)launch_after(gemm_macro_kernel, dim3((unsigned)grid), dim3(NUM_THREADS_MACRO), C::SMEM_BYTES, st, ta, tb, td, margs);
  return cudaGetLastError() == cudaSuccess ? ALTOB200_OK : ALTOB200_ECUDA;
}

static int gemm_macro_common(int64_t M, int64_t N, int64_t K, int32_t num_experts, const void* a_codes,
                             const void* a_scales, const altob200_macro_scale* a_macro, const void* b_codes,
                             const void* b_scales, const altob200_macro_scale* b_macro, const int32_t* group_expert,
                             const int32_t* k_offs, float out_scale, int32_t out_dtype, void* d, int64_t ldd,
                             void* stream) {
  if (a_codes == nullptr || b_codes == nullptr || a_scales == nullptr || b_scales == nullptr || d == nullptr ||
      a_macro == nullptr || b_macro == nullptr || a_macro->codes == nullptr || b_macro->codes == nullptr)
    return ALTOB200_EINVAL_SHAPE;
  if (M <= 0 || N <= 0 || K <= 0 || K % 32 != 0 || ldd < N) return ALTOB200_EINVAL_SHAPE;
  if (group_expert != nullptr && k_offs != nullptr) return ALTOB200_EINVAL_SHAPE;
  if ((group_expert != nullptr || k_offs != nullptr) && num_experts <= 0) return ALTOB200_EINVAL_SHAPE;
  if ((a_macro->row_shift != 0 && a_macro->row_shift != 7) || (b_macro->row_shift != 0 && b_macro->row_shift != 7))
    return ALTOB200_EINVAL_SHAPE;
  const int64_t k_bytes = K / 2;
  if (k_bytes % 16 != 0) return ALTOB200_EINVAL_SHAPE;
  const int osz = out_dtype == ALTOB200_DT_BF16 ? 2 : 4;
  if ((reinterpret_cast<uintptr_t>(a_codes) & 15) || (reinterpret_cast<uintptr_t>(b_codes) & 15) ||
      (reinterpret_cast<uintptr_t>(a_scales) & 15) || (reinterpret_cast<uintptr_t>(b_scales) & 15) ||
      (reinterpret_cast<uintptr_t>(d) & 15) || (ldd * osz) % 16 != 0)
    return ALTOB200_EINVAL_ALIGN;
  const bool row_groups = group_expert != nullptr;
  const int64_t b_rows = N * (row_groups ? num_experts : 1);
  if (M >= (1ll << 31) || b_rows >= (1ll << 31) || k_bytes >= (1ll << 31)) return ALTOB200_ELIMIT;

  CUtensorMap ta, tb, td;
  int rc = make_tmap(&ta, a_codes, M, k_bytes, BM);
  if (rc != ALTOB200_OK) return rc;
  rc = make_tmap(&tb, b_codes, b_rows, k_bytes, CfgMacro::BN);
  if (rc != ALTOB200_OK) return rc;
  // a fold warp stores 32 columns per row: 64 bytes of bf16 (64-byte swizzle) or 128 bytes of fp32
  rc = make_tmap_out(&td, d, k_offs != nullptr ? num_experts : 1, M, N, ldd, out_dtype == ALTOB200_DT_BF16,
                     out_dtype == ALTOB200_DT_BF16 ? 64 : 128);
  if (rc != ALTOB200_OK) return rc;

  MacroGemmArgs m;
  GemmArgs& g = m.g;
  g.M = M; g.N = N; g.K = K; g.k_bytes = k_bytes;
  g.sfa = (const uint8_t*)a_scales; g.sfb = (const uint8_t*)b_scales;
  g.nct = ceil_div(K / 32, 4);
  g.alpha_a = nullptr; g.alpha_b = nullptr;
  g.d = d; g.ldd = ldd; g.out_bf16 = out_dtype == ALTOB200_DT_BF16;
  g.num_experts = row_groups ? num_experts : 0; g.group_expert = group_expert;
  g.sfb_expert_stride = (int64_t)altob200_packed_scale_bytes(N, K / 32);
  g.k_offs = k_offs; g.num_batches = k_offs != nullptr ? num_experts : 1;
  {
    const int64_t tiles_m = ceil_div(M, BM);
    int64_t gm = 8;
    if (gm > tiles_m) gm = tiles_m;
    const int64_t n_groups = ceil_div(tiles_m, gm);
    g.group_m = (int)ceil_div(tiles_m, n_groups);
  }
  g.wait_ns = wait_limit_ns();
  for (int j = 0; j < 4; ++j)
    g.idesc[j] = make_idesc(KIND_MXF4, ALTOB200_FMT_MXFP4, ALTOB200_FMT_MXFP4, BM, CfgMacro::BN, (j & 1) * 2);
#ifdef ALTOB200_GEMM_PROFILE
  {
    const char* e = getenv("ALTOB200_GEMM_DEBUG");
    g.debug = e ? atoi(e) : 0;
  }
#endif
  m.ma.codes = a_macro->codes; m.ma.row_stride = a_macro->row_stride; m.ma.chunk_stride = a_macro->chunk_stride;
  m.ma.expert_stride = 0; m.ma.shift = a_macro->row_shift;
  m.mb.codes = b_macro->codes; m.mb.row_stride = b_macro->row_stride; m.mb.chunk_stride = b_macro->chunk_stride;
  m.mb.expert_stride = row_groups ? b_macro->expert_stride : 0; m.mb.shift = b_macro->row_shift;
  m.out_scale = out_scale;
#ifdef ALTOB200_GEMM_PROFILE
  {
    const char* e = getenv("ALTOB200_MACRO_PROF_PTR");  // device address of the clock table, set by the probe script
    m.prof = e ? reinterpret_cast<unsigned long long*>(strtoull(e, nullptr, 0)) : nullptr;
  }
#endif
  return launch_gemm_macro(ta, tb, td, m, (cudaStream_t)stream);
}

}  // namespace altob200

using namespace altob200;

extern "C" {

int altob200_gemm_blockscaled(int32_t format_a, int32_t format_b, int64_t M, int64_t N, int64_t K,
                              const void* a_codes, const void* a_scales, const void* b_codes,
                              const void* b_scales, const float* alpha_a, const float* alpha_b,
                              int32_t out_dtype, void* d, int64_t ldd, void* stream) {
  return gemm_common(format_a, format_b, M, N, K, 0, a_codes, a_scales, b_codes, b_scales, nullptr, alpha_a,
                     alpha_b, out_dtype, d, ldd, stream);
}

int altob200_grouped_gemm_blockscaled(int32_t format_a, int32_t format_b, int64_t M, int64_t N,
                                      int64_t K, int32_t num_experts, const void* a_codes,
                                      const void* a_scales, const void* b_codes,
                                      const void* b_scales, const int32_t* group_expert,
                                      const float* alpha_a, const float* alpha_b,
                                      int32_t out_dtype, void* d, int64_t ldd, void* stream) {
  if (num_experts <= 0) return ALTOB200_EINVAL_SHAPE;
  return gemm_common(format_a, format_b, M, N, K, num_experts, a_codes, a_scales, b_codes, b_scales,
                     group_expert, alpha_a, alpha_b, out_dtype, d, ldd, stream);
}

int altob200_grouped_gemm_wgrad_blockscaled(int32_t format_a, int32_t format_b, int64_t M, int64_t N, int64_t K,
                                            int32_t num_experts, const void* a_codes, const void* a_scales,
                                            const void* b_codes, const void* b_scales, const int32_t* k_offs,
                                            const float* alpha_a, const float* alpha_b, int32_t out_dtype,
                                            void* d, int64_t ldd, void* stream) {
  if (num_experts <= 0 || k_offs == nullptr) return ALTOB200_EINVAL_SHAPE;
  return gemm_common(format_a, format_b, M, N, K, 0, a_codes, a_scales, b_codes, b_scales, nullptr, alpha_a,
                     alpha_b, out_dtype, d, ldd, stream, k_offs, num_experts);
}

int altob200_gemm_mxfp4_two_level(int64_t M, int64_t N, int64_t K, const void* a_codes, const void* a_scales,
                                  const altob200_macro_scale* a_macro, const void* b_codes, const void* b_scales,
                                  const altob200_macro_scale* b_macro, float out_scale, int32_t out_dtype, void* d,
                                  int64_t ldd, void* stream) {
  return gemm_macro_common(M, N, K, 0, a_codes, a_scales, a_macro, b_codes, b_scales, b_macro, nullptr, nullptr,
                           out_scale, out_dtype, d, ldd, stream);
}

int altob200_grouped_gemm_mxfp4_two_level(int64_t M, int64_t N, int64_t K, int32_t num_experts, const void* a_codes,
                                          const void* a_scales, const altob200_macro_scale* a_macro,
                                          const void* b_codes, const void* b_scales,
                                          const altob200_macro_scale* b_macro, const int32_t* group_expert,
                                          float out_scale, int32_t out_dtype, void* d, int64_t ldd, void* stream) {
  if (num_experts <= 0 || group_expert == nullptr) return ALTOB200_EINVAL_SHAPE;
  return gemm_macro_common(M, N, K, num_experts, a_codes, a_scales, a_macro, b_codes, b_scales, b_macro,
                           group_expert, nullptr, out_scale, out_dtype, d, ldd, stream);
}

int altob200_grouped_gemm_wgrad_mxfp4_two_level(int64_t M, int64_t N, int64_t K, int32_t num_experts,
                                                const void* a_codes, const void* a_scales,
                                                const altob200_macro_scale* a_macro, const void* b_codes,
                                                const void* b_scales, const altob200_macro_scale* b_macro,
                                                const int32_t* k_offs, float out_scale, int32_t out_dtype, void* d,
                                                int64_t ldd, void* stream) {
  if (num_experts <= 0 || k_offs == nullptr) return ALTOB200_EINVAL_SHAPE;
  return gemm_macro_common(M, N, K, num_experts, a_codes, a_scales, a_macro, b_codes, b_scales, b_macro, nullptr,
                           k_offs, out_scale, out_dtype, d, ldd, stream);
}

int altob200_set_wait_limit_ns(uint64_t limit_ns) {
  if (limit_ns == 0) return ALTOB200_EINVAL_SHAPE;
  g_wait_limit_ns.store(limit_ns, std::memory_order_relaxed);
  return ALTOB200_OK;
}

int altob200_selftest_wait_timeout(uint64_t limit_ns, void* stream) {
  if (limit_ns == 0 || limit_ns > 1000000000ull) return ALTOB200_EINVAL_SHAPE;  // at most one second
  wait_selftest_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(limit_ns);
  return cudaGetLastError() == cudaSuccess ? ALTOB200_OK : ALTOB200_ECUDA;
}

int altob200_status_read(void* stream, int32_t detail[4]) {
  cudaStream_t st = (cudaStream_t)stream;
  int h[4] = {0, 0, 0, 0};
  if (cudaStreamSynchronize(st) != cudaSuccess) return ALTOB200_ECUDA;
  if (cudaMemcpyFromSymbol(h, g_status, sizeof(h)) != cudaSuccess) return ALTOB200_ECUDA;
  if (h[0] != 0) {
    const int z[4] = {0, 0, 0, 0};
    if (cudaMemcpyToSymbol(g_status, z, sizeof(z)) != cudaSuccess) return ALTOB200_ECUDA;
  }
  if (detail != nullptr) {
    detail[0] = h[1]; detail[1] = h[2]; detail[2] = h[3]; detail[3] = 0;
  }
  return h[0];
}

}  // extern "C"
