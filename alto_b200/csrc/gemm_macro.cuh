// MXFP4 block-scaled GEMM with two-level ("macro-block") scaling, for sm_100a.
//
//   D[m, n] = out_scale * sum over 128-wide chunks c of K of
//             (1 / fa[m, c]) * (1 / fb[n, c]) * sum_{k in chunk c} A[m, k] * B[n, k]
//
// A and B are MXFP4 operands (E2M1 codes, one E8M0 scale per 32 elements) that were quantised AFTER
// every block of 128 elements along K had been multiplied by a factor in [1, 2) (fa, fb: eight
// mantissa bits each, alto/kernels/fp4/mxfp4/macro_block_scaling.py:70-85).  The factors are not
// powers of two, so they cannot ride on the E8M0 scales of the block-scaled MMA; they are constant
// over a chunk of 128, so the tensor cores accumulate one chunk at a time into tensor memory and
// CUDA cores fold each finished chunk into the running fp32 result, which lives in registers.
// This replaces the reference's emulation of the recipe, dequantise -> descale -> bf16 matmul
// (alto/kernels/fp4/mxfp4/mxfp_linear.py:337-356, mxfp_grouped_gemm/cg_backward.py:668-690).
//
// One CTA (768 threads = six warpgroups, persistent over 128 x 128 output tiles):
//   warpgroup 0   warp 0: producer - per stage (128 bytes of K = two chunks) two tiled TMA loads and the
//                 bulk copies of the stage's scale tiles; warp 1: MMA issuer - two tcgen05.mma per chunk
//                 into one of three 128-column chunk accumulators in tensor memory, then a commit to that
//                 accumulator's "full" barrier; warp 2: waits on the shared-memory barriers for the MMA issuer
//                 and releases it once per CHUNK through a named barrier; warp 3 idle;
//   warpgroup 1   scale transfer shared memory -> tensor memory (as in the plain kernel);
//   warpgroups 2-5  fold + epilogue: sixteen warps, four per tensor-memory lane quarter, each 32 rows x 32
//                 columns of the tile in 32 registers per thread.  Per chunk a warp reads its slice of the
//                 chunk accumulator (one tcgen05.ld), gives the accumulator back, and adds
//                 P * (1/fa[row]) * (1/fb[col]) with packed fp32x2 arithmetic; the column factors of the
//                 chunk pass through a small per-warp shared-memory buffer.  After the last chunk the
//                 registers are scaled, converted, staged and TMA-stored.
// The warpgroups re-divide the register file with setmaxnreg (768 threads x 80 at launch -> 48 for the
// small roles, 96 for the fold warps; the two must balance exactly, see CfgMacro).
// Rows grouped by expert (`group_expert`) and K ranges per batch entry (`k_offs`) work as in the
// plain kernel; every K range starts on a multiple of 128 elements, so chunks never straddle one.
#pragma once
// (included by gemm_sm100.cu inside namespace altob200, after the plain kernels it shares helpers with)

struct MacroSide {
  const uint8_t* codes;     // factor codes: element (row r, chunk c) at ((r >> shift) * row_stride + c * chunk_stride)
  int64_t row_stride, chunk_stride;
  int64_t expert_stride;    // B only: added per expert in row-group mode
  int shift;                // 0: one factor per row; 7: one factor per 128 rows (2-D macro blocks)
};

struct MacroGemmArgs {
  GemmArgs g;
  MacroSide ma, mb;
  float out_scale;
#ifdef ALTOB200_GEMM_PROFILE
  unsigned long long* prof;  // [gridDim.x][4 roles][8] clock sums of a -DALTOB200_GEMM_PROFILE build
#endif
};

// Clock accounting of a profiling build: PROF_NOW() reads the SM clock, PROF_ADD(slot, t0) adds the
// cycles since t0 to a per-thread counter; both vanish from the default build.
#ifdef ALTOB200_GEMM_PROFILE
#define PROF_DECL unsigned long long prof_c[8] = {0, 0, 0, 0, 0, 0, 0, 0}
#define PROF_NOW() clock64()
#define PROF_ADD(slot, t0) prof_c[slot] += (unsigned long long)(clock64() - (t0))
#define PROF_FLUSH(role)                                                                   \
  if (margs.prof != nullptr)                                                               \
    for (int i_ = 0; i_ < 8; ++i_) margs.prof[((size_t)blockIdx.x * 4 + (role)) * 8 + i_] = prof_c[i_]
// event trace of CTA 0: clock of event k of step idx (< 128) of a role, after the per-CTA sums
#define PROF_TRACE(role, idx, k)                                                            \
  if (margs.prof != nullptr && blockIdx.x == 0 && (idx) < 128u)                              \
  margs.prof[(size_t)gridDim.x * 32 + (((role) * 128 + (idx)) * 4 + (k))] = (unsigned long long)clock64()
#else
#define PROF_TRACE(role, idx, k)
#define PROF_DECL
#define PROF_NOW() 0
#define PROF_ADD(slot, t0) (void)(t0)
#define PROF_FLUSH(role)
#endif

constexpr int NUM_THREADS_MACRO = 768;

struct CfgMacro {
  static constexpr int BN = 128;
  static constexpr int SF_TILES = Kind<KIND_MXF4>::SF_TILES;
  static constexpr int A_BYTES = BM * STAGE_K_BYTES;
  static constexpr int B_BYTES = BN * STAGE_K_BYTES;
  static constexpr int SFA_BYTES = SF_TILES * 512;
  static constexpr int SFB_BYTES = SF_TILES * 512;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES + SFA_BYTES + SFB_BYTES;
  static_assert(STAGE_BYTES % 1024 == 0, "stages must keep the 128-byte swizzle atom aligned");
  static constexpr int SF_COLS_A = SF_TILES * 4;
  static constexpr int SF_COLS_B = SF_TILES * 4;
  static constexpr int STAGES = 4;
  static constexpr int P_BUFS = 3;                              // chunk accumulators in tensor memory
  static constexpr int FOLD_WARPS = 16;                         // four per tensor-memory lane quarter, 32 columns each
  static constexpr int FOLD_COLS = BN / (FOLD_WARPS / 4);
  static constexpr int EPI_WARP_BYTES = 4096;                   // bf16: two buffers of 32 rows x 64 bytes; fp32: one of 32 x 128
  static constexpr int EPI_BYTES = FOLD_WARPS * EPI_WARP_BYTES;
  static constexpr int FB_BYTES = FOLD_WARPS * 2 * FOLD_COLS * 4;  // two buffers of 32 column factors per warp
  static constexpr int RCP_BYTES = 256 * 4;                     // 1 / factor for every code
  static constexpr int TMEM_SF_BASE = P_BUFS * BN;
  static constexpr int TMEM_COLS_USED = TMEM_SF_BASE + STAGES * (SF_COLS_A + SF_COLS_B);
  static_assert(TMEM_COLS_USED <= 512, "tensor memory budget");
  static constexpr int NUM_BARS = 3 * STAGES + 2 * P_BUFS;
  static constexpr int SMEM_BYTES =
      STAGES * STAGE_BYTES + EPI_BYTES + FB_BYTES + RCP_BYTES + 1024 /*align*/ + 512 /*barriers*/;
  static_assert(NUM_BARS * 8 + 16 <= 512, "barrier area");
  static_assert(SMEM_BYTES <= 232448, "shared memory budget");
  // Registers per thread after the warpgroups have re-divided the file.  The CTA is launched with 80
  // registers per thread (65536 / 768 rounded down to a multiple of 8, what ptxas reports for this
  // kernel); setmaxnreg.inc can only take what setmaxnreg.dec has released INSIDE the CTA and blocks
  // for ever otherwise, so the two must balance exactly: 2 x 128 x 48 + 4 x 128 x 96 = 768 x 80.
  static constexpr int REGS_LAUNCH = 80;
  static constexpr int REGS_SMALL = 48, REGS_FOLD = 96;
  static_assert(2 * 128 * REGS_SMALL + (FOLD_WARPS / 4) * 128 * REGS_FOLD == NUM_THREADS_MACRO * REGS_LAUNCH,
                "setmaxnreg budget must balance");
  static_assert(NUM_THREADS_MACRO == (8 + FOLD_WARPS) * 32, "role layout");
};

// Tile description plus what the chunk loop needs: the first chunk of the K range, the number of
// chunks, and MMAs per stage limited to the bytes that exist (also without K ranges).
struct MacroTile {
  TileInfo t;
  int64_t chunk0;
  int n_chunks;
  int expert;
};

__device__ __forceinline__ MacroTile decode_macro_tile(const GemmArgs& args, int64_t tile, int64_t tiles_m,
                                                       int64_t tiles_n, int k_stages_dense) {
  MacroTile m;
  m.t = decode_tile<KIND_MXF4, CfgMacro::BN>(args, tile, tiles_m, tiles_n, k_stages_dense);
  m.expert = 0;
  int64_t bytes = args.k_bytes;
  m.chunk0 = 0;
  if (args.k_offs != nullptr) {
    const int64_t e = m.t.batch;
    const int64_t k0 = e > 0 ? __ldg(args.k_offs + e - 1) : 0;
    const int64_t k1 = __ldg(args.k_offs + e);
    bytes = (k1 - k0) / 2;
    m.chunk0 = k0 >> 7;
  } else {
    const int64_t tail = bytes - (int64_t)(m.t.k_stages - 1) * STAGE_K_BYTES;
    m.t.last_mmas = (int)((tail + 31) / 32);
    if (args.num_experts > 0 && !m.t.skip) m.expert = __ldg(args.group_expert + m.t.mb);
  }
  m.n_chunks = bytes > 0 ? (int)((bytes + 63) / 64) : 0;
  return m;
}

// acc += P * (ra * fb[col]) for the 32 columns of one chunk that a fold warp owns (P: raw tensor-memory
// words of this thread's row)
__device__ __forceinline__ void fold_cols(float2 (&acc)[16], const uint32_t (&p)[32], float ra, const float* fb,
                                          bool b_uniform, float rb_uniform) {
  if (b_uniform) {
    const float g = __fmul_rn(ra, rb_uniform);
    const float2 g2 = make_float2(g, g);
#pragma unroll
    for (int j = 0; j < 16; ++j)
      acc[j] = __ffma2_rn(make_float2(u2f(p[2 * j]), u2f(p[2 * j + 1])), g2, acc[j]);
  } else {
    const float2 ra2 = make_float2(ra, ra);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float4 f = *reinterpret_cast<const float4*>(fb + 4 * j);
      const float2 g0 = __fmul2_rn(ra2, make_float2(f.x, f.y));
      const float2 g1 = __fmul2_rn(ra2, make_float2(f.z, f.w));
      acc[2 * j] = __ffma2_rn(make_float2(u2f(p[4 * j]), u2f(p[4 * j + 1])), g0, acc[2 * j]);
      acc[2 * j + 1] = __ffma2_rn(make_float2(u2f(p[4 * j + 2]), u2f(p[4 * j + 3])), g1, acc[2 * j + 1]);
    }
  }
}

__global__ void __launch_bounds__(NUM_THREADS_MACRO, 1)
gemm_macro_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                  const __grid_constant__ CUtensorMap tmap_d, const MacroGemmArgs margs) {
  using C = CfgMacro;
  constexpr int BN = C::BN;
  const GemmArgs& args = margs.g;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* epi = smem + C::STAGES * C::STAGE_BYTES;
  float* fb_all = reinterpret_cast<float*>(epi + C::EPI_BYTES);
  float* rcp_tab = reinterpret_cast<float*>(epi + C::EPI_BYTES + C::FB_BYTES);
  uint64_t* bars = reinterpret_cast<uint64_t*>(epi + C::EPI_BYTES + C::FB_BYTES + C::RCP_BYTES);
  uint64_t* full_bar = bars;
  uint64_t* empty_bar = bars + C::STAGES;
  uint64_t* sf_full = bars + 2 * C::STAGES;
  uint64_t* p_full = bars + 3 * C::STAGES;
  uint64_t* p_empty = p_full + C::P_BUFS;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(p_empty + C::P_BUFS);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t tiles_m = (args.M + BM - 1) / BM;
  const int64_t tiles_n = (args.N + BN - 1) / BN;
  const int64_t n_tiles = tiles_m * tiles_n * (args.k_offs != nullptr ? args.num_batches : 1);
  const int k_stages = (int)((args.k_bytes + STAGE_K_BYTES - 1) / STAGE_K_BYTES);

  if (threadIdx.x == 0) {
    for (int s = 0; s < C::STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
      mbar_init(&sf_full[s], 4);
    }
    for (int p = 0; p < C::P_BUFS; ++p) {
      mbar_init(&p_full[p], 1);
      mbar_init(&p_empty[p], C::FOLD_WARPS);
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  // scale staging starts from zero: a ragged last stage never feeds uninitialised scale bytes
  for (int s = 0; s < C::STAGES; ++s) {
    uint32_t* z = reinterpret_cast<uint32_t*>(smem + s * C::STAGE_BYTES + C::A_BYTES + C::B_BYTES);
    for (int i = threadIdx.x; i < (C::SFA_BYTES + C::SFB_BYTES) / 4; i += NUM_THREADS_MACRO) z[i] = 0u;
  }
  // 1 / factor(code), factor = 1 + code / 256 (exact), correctly rounded
  if (threadIdx.x < 256) rcp_tab[threadIdx.x] = __frcp_rn(u2f((threadIdx.x << 15) + (127u << 23)));
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
  grid_dependency_wait();   // set-up done; global memory from here on (programmatic dependent launch)

  if (warp < 4) {
    setmaxnreg_dec<C::REGS_SMALL>();
    // Producer and MMA issuer: the WHOLE warp runs the loop and waits on the barriers, one elected lane
    // issues the TMA / tcgen05 instructions.  Those instructions take their operands (descriptors,
    // addresses, coordinates) from uniform registers; computed by a converged warp from kernel parameters
    // and loop counters they are uniform values from the start, whereas the same arithmetic inside an
    // `if (lane == 0)` region yields per-thread values that have to be moved to uniform registers one by
    // one in front of every instruction (measured: ~270 cycles per tcgen05.mma).
    if (warp == 0) {
      // ------------------------------ producer ------------------------------
      const bool elected = elect_one();
      uint32_t it = 0;
      bool alive = true;
      PROF_DECL;
      const long long t_all = PROF_NOW();
      for (int64_t tile = blockIdx.x; tile < n_tiles && alive; tile += gridDim.x) {
        const MacroTile mt = decode_macro_tile(args, tile, tiles_m, tiles_n, k_stages);
        const TileInfo& ti = mt.t;
        if (ti.skip) continue;
        const int64_t mb = ti.mb, nb = ti.nb;
        for (int ks = 0; ks < ti.k_stages; ++ks, ++it) {
          const int s = it % C::STAGES;
          const long long t0 = PROF_NOW();
          alive = __all_sync(0xFFFFFFFFu,
                             mbar_wait(&empty_bar[s], ((it / C::STAGES) & 1) ^ 1, abort_flag, 21, args.wait_ns));
          if (!alive) break;
          PROF_ADD(1, t0);
          if (lane == 0) { PROF_TRACE(0, it, 0); }
          uint8_t* st = smem + s * C::STAGE_BYTES;
          const int64_t cb0 = ti.sf_tile0 + (int64_t)ks * C::SF_TILES;
          int64_t sf_tiles = args.nct - cb0;
          if (sf_tiles > C::SF_TILES) sf_tiles = C::SF_TILES;
          const uint32_t sf_bytes = (uint32_t)sf_tiles * 512u;
          const int32_t kx = (int32_t)(ti.k_byte0 + (int64_t)ks * STAGE_K_BYTES);
          if (ALTOB200_DBG(args, 4) && it >= (uint32_t)C::STAGES) {
            if (elected) mbar_arrive(&full_bar[s]);
            continue;
          }
          if (elected) {
            mbar_expect_tx(&full_bar[s], C::A_BYTES + C::B_BYTES + 2 * sf_bytes);
            tma_load_2d(st, &tmap_a, kx, (int32_t)(mb * BM), &full_bar[s]);
            tma_load_2d(st + C::A_BYTES, &tmap_b, kx, (int32_t)ti.b_row0, &full_bar[s]);
            bulk_load(st + C::A_BYTES + C::B_BYTES, args.sfa + (mb * args.nct + cb0) * 512, sf_bytes, &full_bar[s]);
            bulk_load(st + C::A_BYTES + C::B_BYTES + C::SFA_BYTES, ti.sfb + (nb * args.nct + cb0) * 512, sf_bytes,
                      &full_bar[s]);
          }
        }
      }
      PROF_ADD(0, t_all);
      if (lane == 0) { PROF_FLUSH(0); }
    } else if (warp == 1) {
      // ------------------------------ MMA issuer ------------------------------
      // Never waits on a shared-memory barrier itself (such a wait between two tcgen05.mma costs ~150
      // cycles during which the tensor pipe idles): warp 2 waits and meets this warp at named barrier
      // 1 + stage.
      const bool elected = elect_one();
      uint32_t it = 0, pc = 0;
      bool alive = true;
      const uint32_t smem_base = smem_u32(smem);
      PROF_DECL;
      const long long t_all = PROF_NOW();
      for (int64_t tile = blockIdx.x; tile < n_tiles && alive; tile += gridDim.x) {
        const MacroTile mt = decode_macro_tile(args, tile, tiles_m, tiles_n, k_stages);
        const TileInfo& ti = mt.t;
        if (ti.skip) continue;
        for (int ks = 0; ks < ti.k_stages; ++ks, ++it) {
          const int n_mma = (ks == ti.k_stages - 1) ? ti.last_mmas : 4;
          const int s = it % C::STAGES;
          const uint32_t st4 = (smem_base + (uint32_t)s * C::STAGE_BYTES) >> 4;
          const uint32_t sfa_t = tmem_base + C::TMEM_SF_BASE + s * (C::SF_COLS_A + C::SF_COLS_B);
          const uint32_t sfb_t = sfa_t + C::SF_COLS_A;
          const uint32_t a_lo = st4 | 0x10000u;
          const uint32_t b_lo = a_lo + (C::A_BYTES >> 4);
          // The issuer is released per chunk (two MMAs), not per stage: a stage holds two chunks and only
          // three chunk accumulators exist, so a release per stage would wait for the fold of the previous
          // stage's FIRST chunk and leave one chunk of overlap instead of three.
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            if (2 * h >= n_mma) break;
            const long long t0 = PROF_NOW();
            // operands and scales of the stage are in place and this chunk's accumulator is drained
            if (named_barrier_or(1 + 2 * s + h, 64, false)) { alive = false; break; }
            PROF_ADD(1, t0);
            tc_fence_after();
            const uint32_t buf = pc % C::P_BUFS;
            if (elected) {
#pragma unroll
              for (int j = 2 * h; j < 2 * h + 2; ++j) {
                if (j < n_mma)
                  tc_mma<KIND_MXF4>(tmem_base + buf * BN, desc_of(DESC_SW128_HI, a_lo + 2 * j),
                                    desc_of(DESC_SW128_HI, b_lo + 2 * j), args.idesc[j], (uint32_t)(j & 1),
                                    sfa_t + h * 4, sfb_t + h * 4);
              }
              tc_commit(&p_full[buf]);
              if (2 * h + 2 >= n_mma) tc_commit(&empty_bar[s]);
            }
            __syncwarp();
            ++pc;
          }
          if (!alive) break;
        }
      }
      PROF_ADD(0, t_all);
      if (lane == 0) { PROF_FLUSH(1); }
    } else if (warp == 2) {
      // ------------------------------ wait warp ------------------------------
      uint32_t it = 0, pc = 0;
      bool alive = true;
      for (int64_t tile = blockIdx.x; tile < n_tiles && alive; tile += gridDim.x) {
        const MacroTile mt = decode_macro_tile(args, tile, tiles_m, tiles_n, k_stages);
        const TileInfo& ti = mt.t;
        if (ti.skip) continue;
        for (int ks = 0; ks < ti.k_stages; ++ks, ++it) {
          const int n_mma = (ks == ti.k_stages - 1) ? ti.last_mmas : 4;
          const int n_chunks = (n_mma + 1) >> 1;
          const int s = it % C::STAGES;
          bool ok = mbar_wait(&full_bar[s], (it / C::STAGES) & 1, abort_flag, 23, args.wait_ns);
          ok = ok && mbar_wait(&sf_full[s], (it / C::STAGES) & 1, abort_flag, 25, args.wait_ns);
          for (int c = 0; c < n_chunks && alive; ++c, ++pc) {
            ok = ok && mbar_wait(&p_empty[pc % C::P_BUFS], ((pc / C::P_BUFS) & 1) ^ 1, abort_flag, 22, args.wait_ns);
            const bool failed = !__all_sync(0xFFFFFFFFu, ok);
            if (named_barrier_or(1 + 2 * s + c, 64, failed)) alive = false;
          }
          if (!alive) break;
        }
      }
    }
  } else if (warp < 8) {
    // ------------------------------ scale transfer ------------------------------
    setmaxnreg_dec<C::REGS_SMALL>();
    const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
    uint32_t it = 0;
    bool alive = true;
    PROF_DECL;
    const long long t_all = PROF_NOW();
    for (int64_t tile = blockIdx.x; tile < n_tiles && alive; tile += gridDim.x) {
      const MacroTile mt = decode_macro_tile(args, tile, tiles_m, tiles_n, k_stages);
      const TileInfo& ti = mt.t;
      if (ti.skip) continue;
      for (int ks = 0; ks < ti.k_stages; ++ks, ++it) {
        const int s = it % C::STAGES;
        const long long t0 = PROF_NOW();
        if (!mbar_wait(&full_bar[s], (it / C::STAGES) & 1, abort_flag, 26, args.wait_ns)) { alive = false; break; }
        PROF_ADD(1, t0);
        if (warp == 4 && lane == 0) { PROF_TRACE(2, it, 0); }
        const uint8_t* sf = smem + s * C::STAGE_BYTES + C::A_BYTES + C::B_BYTES + lane * 16;
        const uint32_t sfa_t = tmem_base + lane_base + C::TMEM_SF_BASE + s * (C::SF_COLS_A + C::SF_COLS_B);
        const uint32_t sfb_t = sfa_t + C::SF_COLS_A;
        if (!(ALTOB200_DBG(args, 1) && it > 0)) {
#pragma unroll
          for (int t = 0; t < C::SF_TILES; ++t) {
            const uint4 a = *reinterpret_cast<const uint4*>(sf + t * 512);
            tc_st4(sfa_t + t * 4, a.x, a.y, a.z, a.w);
            const uint4 b = *reinterpret_cast<const uint4*>(sf + C::SFA_BYTES + t * 512);
            tc_st4(sfb_t + t * 4, b.x, b.y, b.z, b.w);
          }
          tc_wait_st();
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&sf_full[s]);
        if (warp == 4 && lane == 0) { PROF_TRACE(2, it, 1); }
      }
    }
    PROF_ADD(0, t_all);
    if (warp == 4 && lane == 0) { PROF_FLUSH(2); }
  } else {
    // ------------------------------ fold + epilogue ------------------------------
    // Sixteen warps, four per tensor-memory lane quarter, each 32 rows x 32 columns of the tile.  What
    // bounds the fold is the latency of the tensor-memory load (a warp has one in flight and waits for
    // it), so the chunk is spread over as many warps as the register file carries: 64 KB per chunk are
    // in flight at once, and the four warps of a scheduler cover each other's waits.
    setmaxnreg_inc<C::REGS_FOLD>();
    constexpr int FC = C::FOLD_COLS;
    const int quad = warp & 3;                        // tensor-memory lane quarter this warp may read
    const int cq = (warp - 8) >> 2;                   // columns [32 cq, 32 cq + 32) of the tile
    const int fold_idx = warp - 8;
    uint8_t* epi_warp = epi + fold_idx * C::EPI_WARP_BYTES;
    float* fb_warp = fb_all + fold_idx * (2 * FC);
    const bool b_uniform = margs.mb.shift >= 7;       // one B factor per 128-column tile and chunk
    const bool out_bf16 = args.out_bf16 != 0;
    const uint32_t t_row = tmem_base + ((uint32_t)(quad * 32) << 16) + cq * FC;
    uint32_t pc = 0, store_it = 0;
    uint32_t p_buf = 0, p_phase = 0;                  // position in the ring of chunk accumulators, its phase
    bool alive = true;
    PROF_DECL;
    const long long t_all = PROF_NOW();
    for (int64_t tile = blockIdx.x; tile < n_tiles && alive; tile += gridDim.x) {
      const MacroTile mt = decode_macro_tile(args, tile, tiles_m, tiles_n, k_stages);
      const TileInfo& ti = mt.t;
      float2 acc[FC / 2];
#pragma unroll
      for (int j = 0; j < FC / 2; ++j) acc[j] = make_float2(0.0f, 0.0f);
      if (!ti.skip) {
        // factor codes of this thread's row of A and of the column of B this lane stages
        int64_t m = ti.mb * BM + quad * 32 + lane;
        if (m >= args.M) m = args.M - 1;
        int64_t n0 = ti.nb * BN + cq * FC + lane;
        if (n0 >= args.N) n0 = args.N - 1;
        const uint8_t* pa = margs.ma.codes + (m >> margs.ma.shift) * margs.ma.row_stride +
                            mt.chunk0 * margs.ma.chunk_stride;
        const uint8_t* pb = margs.mb.codes + (int64_t)mt.expert * margs.mb.expert_stride +
                            mt.chunk0 * margs.mb.chunk_stride + (n0 >> margs.mb.shift) * margs.mb.row_stride;
        const int nch = mt.n_chunks;
        uint32_t ca = __ldg(pa), cb = __ldg(pb);
        uint32_t p[FC];   // chunk accumulator words of this thread's row
        // The loop body is what bounds the kernel (instruction issue of sixteen of these warps), so the
        // ring position and its phase are carried instead of divided out, the code pointers advance by
        // their strides, and the two barrier addresses are 32-bit shared-memory addresses.
        const int64_t sa = margs.ma.chunk_stride, sb = margs.mb.chunk_stride;
        for (int c = 0; c < nch; ++c) {
          if (ALTOB200_DBG(args, 256)) continue;
          long long t0 = PROF_NOW();
          alive = mbar_wait(&p_full[p_buf], p_phase, abort_flag, 24, args.wait_ns);
          PROF_ADD(2, t0);
          if (!alive) break;
          tc_fence_after();
          if (warp == 8 && lane == 0) { PROF_TRACE(3, pc, 0); }
          tc_ld32(t_row + p_buf * BN, p);
          // under the load: this chunk's factors, the next chunk's codes
          t0 = PROF_NOW();
          const float ra = rcp_tab[ca], rb = rcp_tab[cb];
          pa += sa;
          pb += sb;
          if (c + 1 < nch) {
            ca = __ldg(pa);
            cb = __ldg(pb);
          }
          float* fb = fb_warp + (c & 1) * FC;
          if (!b_uniform) {
            fb[lane] = rb;
            __syncwarp();
          }
          PROF_ADD(6, t0);
          t0 = PROF_NOW();
          tc_wait_ld();                 // the chunk has left tensor memory
          PROF_ADD(1, t0);
          t0 = PROF_NOW();
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(&p_empty[p_buf]);
          if (warp == 8 && lane == 0) { PROF_TRACE(3, pc, 1); }
          ++pc;
          if (++p_buf == C::P_BUFS) {
            p_buf = 0;
            p_phase ^= 1u;
          }
          PROF_ADD(7, t0);
          if (ALTOB200_DBG(args, 64)) continue;   // profiling builds only: chunks are handed straight back
          t0 = PROF_NOW();
          fold_cols(acc, p, ra, fb, b_uniform, rb);
          PROF_ADD(3, t0);
        }
        if (!alive) break;
      }
      // ---- epilogue of the tile: this warp's 32 rows x 32 columns ----
      const long long t_epi = PROF_NOW();
      const float os = margs.out_scale;
      const int64_t row0 = ti.mb * BM + quad * 32;
      const int64_t col0 = ti.nb * BN + cq * FC;
      uint32_t buf;
      if (out_bf16) {
        // 64-byte rows (64-byte swizzle: chunk index ^ bits 1-2 of the row), two buffers
        if (lane == 0) bulk_wait_read<1>();  // the store issued two tiles ago has finished reading this buffer
        __syncwarp();
        buf = (store_it & 1u) * 2048u;
        const uint32_t row = smem_u32(epi_warp) + buf + (uint32_t)lane * 64u;
        const uint32_t sw = (uint32_t)((lane >> 1) & 3);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          uint32_t o[4];
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            const float2 v = acc[4 * j + q];
            const __nv_bfloat162 p2 = __floats2bfloat162_rn(__fmul_rn(v.x, os), __fmul_rn(v.y, os));
            o[q] = *reinterpret_cast<const uint32_t*>(&p2);
          }
          st_shared_v4(row + ((((uint32_t)j) ^ sw) << 4), o[0], o[1], o[2], o[3]);
        }
      } else {
        // 128-byte rows (128-byte swizzle), one buffer
        if (lane == 0) bulk_wait_read<0>();
        __syncwarp();
        buf = 0u;
        const uint32_t row = smem_u32(epi_warp) + (uint32_t)lane * 128u;
        const uint32_t sw = (uint32_t)(lane & 7);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float2 v0 = acc[2 * j], v1 = acc[2 * j + 1];
          st_shared_v4(row + ((((uint32_t)j) ^ sw) << 4), f2u(__fmul_rn(v0.x, os)), f2u(__fmul_rn(v0.y, os)),
                       f2u(__fmul_rn(v1.x, os)), f2u(__fmul_rn(v1.y, os)));
        }
      }
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      __syncwarp();
      if (lane == 0) {
        if (row0 < args.M && col0 < args.N)
          tma_store_3d(epi_warp + buf, &tmap_d, (int32_t)col0, (int32_t)row0, ti.batch);
        bulk_commit();  // one group per tile, empty or not: the waits above count groups
      }
      ++store_it;
      PROF_ADD(5, t_epi);
    }
    if (lane == 0) bulk_wait_all();
    PROF_ADD(0, t_all);
    if (warp == 8 && lane == 0) { PROF_FLUSH(3); }
  }

  // ------------------------------ teardown ------------------------------
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, 512;" ::"r"(tmem_base) : "memory");
  }
}
