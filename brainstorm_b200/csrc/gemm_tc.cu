// Tensor-core GEMM of the B200 handler: out (+)= op(a) . op(b) in fp32 accuracy on
// the 5th-generation tensor cores.
//
//  * Operand tiles are brought into shared memory by TMA (cp.async.bulk.tensor,
//    128-byte swizzle) straight from the caller's row-major arrays; all four
//    transpose combinations map to K-major or MN-major UMMA operands, so no
//    operand is ever transposed or copied in global memory.
//  * tcgen05.mma kind::tf32 reads only the upper 19 bits of each fp32 value.  To
//    keep fp32-level accuracy every product is split 3xTF32:
//        a = a_hi + a_lo,  b = b_hi + b_lo   (a_hi = a with 13 low bits cleared)
//        a.b ~= a_lo.b_hi + a_hi.b_lo + a_hi.b_hi      (fp32 accumulate in TMEM)
//    The low parts are produced on the fly: four warps turn each landed tile into
//    its residual tile in a second shared-memory buffer with the same swizzled
//    layout (the transform is elementwise, so the layout never matters).
//  * The tensor core adds into its fp32 accumulator with truncation, not rounding:
//    left alone, a long K loop loses about 2e-8 * K of the result's magnitude.  The
//    accumulation in TMEM is therefore cut into chunks of 128 along K; each finished
//    chunk is drained into fp32 registers (round-to-nearest adds) while the MMAs of
//    the next chunk run on the second TMEM buffer.
//  * Warp roles (320 threads): warp 0 = TMA producer, warp 1 = MMA issuer and TMEM
//    owner, warps 2-5 = split transform, warps 6-9 = chunk drain and epilogue
//    (TMEM -> registers -> global, optional += C).
//  * Every mbarrier wait is bounded.  On a timeout the CTA raises a flag in
//    host-visible memory, skips its stores, drains its own TMA copies, frees its
//    TMEM and returns; the host reports the flag at the next synchronisation.
//
// Roofline: tensor pipe.  2*M*N*K useful flops cost 3x that in TF32 MMAs.
#include <cuda.h>

#include <mutex>
#include <unordered_map>

#include "common.cuh"

namespace b200 {

constexpr int TC_BM = 128;
constexpr int TC_BK = 32;               // 32 fp32 = one 128-byte swizzle row
constexpr int TC_THREADS = 320;
constexpr int TC_CHUNK_KB = 4;            // k-blocks per TMEM accumulation chunk (128 along K)
constexpr uint32_t TC_SPIN_LIMIT = 1u << 22;

// ---- PTX wrappers --------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ uint32_t mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok;
}
// Non-blocking phase test (try_wait may suspend the thread for a while).
__device__ __forceinline__ uint32_t mbar_test_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok;
}
// Bounded wait.  Returns false (and raises *abort_flag) if the phase did not
// complete within the spin limit or another role already gave up.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
  for (uint32_t it = 0; it < TC_SPIN_LIMIT; ++it) {
    if (mbar_try_wait(bar, parity)) return true;
    if (it > 64) {
      if (*abort_flag) return false;
      __nanosleep(it > 4096 ? 256 : 32);
    }
  }
  *abort_flag = 1;
  return false;
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int c0, int c1,
                                            uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(bar)
      : "memory");
}
__device__ __forceinline__ void tmem_alloc(uint32_t slot, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(slot), "r"(cols) : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void mma_tf32(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                         uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void mma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, float* v) {
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

// Shared-memory matrix descriptor of a 128-byte-swizzled operand tile.
//  K-major : rows of 32 fp32 (128 B) along K, one row per M/N index; 8-row groups
//            1024 B apart (SBO); LBO unused.  Swizzle: 16-byte chunks XOR row%8
//            (layout type 2, TMA SWIZZLE_128B).
//  MN-major: boxes of [32 K-rows][32 fp32 along M/N]; boxes 4096 B apart (LBO),
//            4-row K groups 512 B apart (SBO).  32-bit MN-major operands exist only
//            in the 32-byte-atom flavour of the 128-byte swizzle: 32-byte chunks XOR
//            row%4 (layout type 1, TMA SWIZZLE_128B_ATOM_32B).
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr, uint32_t lbo_bytes, uint32_t sbo_bytes,
                                              uint32_t layout_type) {
  uint64_t d = 0;
  d |= (uint64_t)((addr >> 4) & 0x3FFF);
  d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFF) << 16;
  d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFF) << 32;
  d |= (uint64_t)1 << 46;  // descriptor version (Blackwell)
  d |= (uint64_t)layout_type << 61;
  return d;
}

template <int BN>
struct TcConfig {
  static constexpr int A_BYTES = TC_BM * TC_BK * 4;                      // 16 KiB
  static constexpr int B_BYTES = BN * TC_BK * 4;
  static constexpr int STAGE_BYTES = 2 * (A_BYTES + B_BYTES);            // hi + lo of both
  static constexpr int STAGES = (BN >= 256) ? 2 : (BN >= 128) ? 3 : (BN >= 64) ? 4 : 5;
  // Tiles of up to 128 columns keep the two small terms of the split (lo.hi, hi.lo) in an
  // accumulator of their own: the tensor core truncates its accumulator at every MMA, and an
  // addition of a small term to the large running sum loses as much as an addition of a
  // large one.  Apart, only the hi.hi MMAs (a third of them) round at the large magnitude.
  // 256-wide tiles have no tensor-memory columns left for it.
  static constexpr bool SPLIT_ACC = BN <= 128;
  static constexpr int TMEM_COLS = (SPLIT_ACC ? 4 : 2) * BN;             // two buffers of one or two accumulators
  // Register accumulators per thread are capped at 128: a 256-wide tile is drained by
  // two groups of four warps (the split-transform warps take columns [0, 128), the
  // drain warps [128, 256)); narrower tiles by the drain warps alone.
  static constexpr int DRAIN_GROUPS = (BN > 128) ? 2 : 1;
  static constexpr int ACC = BN / DRAIN_GROUPS;
  // the epilogue stages each warp's 32 x ACC tile (padded) in the then idle stage memory
  static_assert(4 * DRAIN_GROUPS * 32 * (ACC + 4) * 4 <= STAGES * STAGE_BYTES, "epilogue staging does not fit");
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*align slack*/ + 256 /*barriers*/;
};

// The residual of the TF32 truncation, exact in fp32.
__device__ __forceinline__ float tf32_residual(float x) {
  return x - __uint_as_float(__float_as_uint(x) & 0xFFFFE000u);
}

// Residual tile of a landed tile, done by 128 threads: lo[i] = residual(hi[i]) for the
// NV float4 of this thread (thread t owns float4 t, t + 128, ...).  All loads of a batch
// of eight are issued before the first store, so their latencies overlap (the compiler
// cannot reorder them itself: the two buffers may alias for all it knows).
// Measured and not kept: rounding the residual to the nearest TF32 value before the store
// (the tensor core truncates it otherwise) moves the bias of a product by 2e-7 and costs 8 %
// of the kernel's throughput; rounding the landed tile itself to the nearest TF32 value and
// writing it back (residuals of either sign) halves the bias and costs 30 %.
template <int NV>
__device__ __forceinline__ void split_tile(const float4* __restrict__ hi, float4* __restrict__ lo, int t) {
  constexpr int BATCH = NV < 8 ? NV : 8;
  static_assert(NV % BATCH == 0, "tile size");
#pragma unroll
  for (int i0 = 0; i0 < NV; i0 += BATCH) {
    float4 v[BATCH];
#pragma unroll
    for (int i = 0; i < BATCH; ++i) v[i] = hi[t + 128 * (i0 + i)];
#pragma unroll
    for (int i = 0; i < BATCH; ++i)
      lo[t + 128 * (i0 + i)] = make_float4(tf32_residual(v[i].x), tf32_residual(v[i].y), tf32_residual(v[i].z),
                                           tf32_residual(v[i].w));
  }
}

// acc[0..NCOLS) += the NCOLS accumulator columns at taddr of this warp's TMEM lanes
template <int NCOLS>
__device__ __forceinline__ void drain_add(uint32_t taddr, float (&acc)[NCOLS]) {
#pragma unroll
  for (int cc = 0; cc < NCOLS / 32; ++cc) {
    float v[32];
    tmem_ld32(taddr + (uint32_t)(cc * 32), v);
#pragma unroll
    for (int j = 0; j < 32; ++j) acc[cc * 32 + j] += v[j];
  }
}

// Epilogue of one warp: its 32 rows x NCOLS accumulators (one row per lane) go to
// c[(row0 + r) * ldc + col0 + j] (+= when accumulating).  A lane-per-row store would
// touch 32 different lines per instruction and serialise in the load/store unit, so
// the tile is first transposed through shared memory (sbuf: 32 x (NCOLS + 4) floats,
// conflict-free) and then written row by row with whole-line stores.
template <int NCOLS>
__device__ __forceinline__ void store_tile(const float (&acc)[NCOLS], float* sbuf, float* c, int64_t ldc,
                                           int row0, int col0, int M, int N, int accumulate) {
  constexpr int LD = NCOLS + 4;
  constexpr int V = NCOLS / 4;               // float4 groups per row
  const int lane = threadIdx.x & 31;
#pragma unroll
  for (int j = 0; j < NCOLS; j += 4)
    *reinterpret_cast<float4*>(sbuf + lane * LD + j) = make_float4(acc[j], acc[j + 1], acc[j + 2], acc[j + 3]);
  __syncwarp();
  const bool vec_ok = ((reinterpret_cast<uintptr_t>(c) & 15) == 0) && (ldc % 4 == 0);
#pragma unroll 4
  for (int idx = lane; idx < 32 * V; idx += 32) {
    const int r = idx / V, g = idx - r * V;
    const int row = row0 + r, col = col0 + 4 * g;
    if (row >= M || col >= N) continue;
    float4 o = *reinterpret_cast<const float4*>(sbuf + r * LD + 4 * g);
    float* p = c + (int64_t)row * ldc + col;
    if (vec_ok && col + 4 <= N) {
      if (accumulate) {
        const float4 old = *reinterpret_cast<const float4*>(p);
        o.x += old.x; o.y += old.y; o.z += old.z; o.w += old.w;
      }
      *reinterpret_cast<float4*>(p) = o;
    } else {
      const float v[4] = {o.x, o.y, o.z, o.w};
#pragma unroll
      for (int j = 0; j < 4; ++j)
        if (col + j < N) p[j] = accumulate ? p[j] + v[j] : v[j];
    }
  }
}

template <int BN>
__global__ void __launch_bounds__(TC_THREADS, 1)
gemm_tf32x3_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                   float* __restrict__ c, int M, int N, int K, int64_t ldc, int accumulate,
                   int a_mn_major, int b_mn_major, int* error_flag, int kb_per_split,
                   int64_t split_stride, int chunk_kb) {
  using Cfg = TcConfig<BN>;
  constexpr int S = Cfg::STAGES;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + S * Cfg::STAGE_BYTES);
  // bars[0..S) full, [S..2S) split, [2S..3S) empty, [3S..3S+2) chunk ready, [3S+2..3S+4) chunk drained
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 3 * S + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m0 = blockIdx.y * TC_BM, n0 = blockIdx.x * BN;
  // split-K: CTA z covers k-blocks [kb_begin, kb_begin + num_kb) and writes its own
  // partial result at c + z * split_stride
  const int kb_begin = blockIdx.z * kb_per_split;
  const int num_kb = min((K + TC_BK - 1) / TC_BK - kb_begin, kb_per_split);
  c += (int64_t)blockIdx.z * split_stride;
  const uint32_t bar0 = smem_u32(bars);
  auto full_bar = [&](int s) { return bar0 + 8u * s; };
  auto split_bar = [&](int s) { return bar0 + 8u * (S + s); };
  auto empty_bar = [&](int s) { return bar0 + 8u * (2 * S + s); };
  auto acc_full_bar = [&](int b) { return bar0 + 8u * (3 * S + b); };
  auto acc_empty_bar = [&](int b) { return bar0 + 8u * (3 * S + 2 + b); };
  const uint32_t smem_base = smem_u32(smem);
  auto a_hi = [&](int s) { return smem_base + s * Cfg::STAGE_BYTES; };
  auto a_lo = [&](int s) { return a_hi(s) + Cfg::A_BYTES; };
  auto b_hi = [&](int s) { return a_hi(s) + 2 * Cfg::A_BYTES; };
  auto b_lo = [&](int s) { return b_hi(s) + Cfg::B_BYTES; };

  if (threadIdx.x == 0) {
    for (int s = 0; s < S; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(split_bar(s), 128);
      mbar_init(empty_bar(s), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(acc_full_bar(b), 1);
      mbar_init(acc_empty_bar(b), 128 * Cfg::DRAIN_GROUPS);
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  pdl_launch_dependents();
  if (warp == 0 && lane == 0) {   // fetch the two TMA descriptors while the prologue runs
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_a) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_b) : "memory");
  }
  if (warp == 1) tmem_alloc(smem_u32(tmem_slot), Cfg::TMEM_COLS);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_d = *tmem_slot;
  // everything above touched only this CTA's shared and tensor memory; operands and
  // the output may still be in use by the previous kernel of the stream
  pdl_wait();

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      int issued = 0;
      for (int kb = 0; kb < num_kb; ++kb) {
        const int s = kb % S;
        const uint32_t ph = (kb / S) & 1;
        if (!mbar_wait(empty_bar(s), ph ^ 1, abort_flag)) break;
        mbar_expect_tx(full_bar(s), Cfg::A_BYTES + Cfg::B_BYTES);
        const int k0 = (kb_begin + kb) * TC_BK;
        if (!a_mn_major) {
          tma_load_2d(a_hi(s), &map_a, k0, m0, full_bar(s));
        } else {
#pragma unroll
          for (int j = 0; j < TC_BM / 32; ++j)
            tma_load_2d(a_hi(s) + j * (TC_BK * 128), &map_a, m0 + 32 * j, k0, full_bar(s));
        }
        if (!b_mn_major) {
          tma_load_2d(b_hi(s), &map_b, k0, n0, full_bar(s));
        } else {
#pragma unroll
          for (int j = 0; j < BN / 32; ++j)
            tma_load_2d(b_hi(s) + j * (TC_BK * 128), &map_b, n0 + 32 * j, k0, full_bar(s));
        }
        issued = kb + 1;
      }
      if (*abort_flag) {
        // drain: copies already issued must land before shared memory is released
        const int first = issued > S ? issued - S : 0;
        for (int kb = first; kb < issued; ++kb) {
          const uint32_t bar = full_bar(kb % S), ph = (kb / S) & 1;
          for (uint32_t it = 0; it < TC_SPIN_LIMIT && !mbar_try_wait(bar, ph); ++it) __nanosleep(64);
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    // instruction descriptor: D = F32, A = B = TF32, majors, N >> 3, M >> 4
    const uint32_t idesc = (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(a_mn_major != 0) << 15) |
                           ((uint32_t)(b_mn_major != 0) << 16) | ((uint32_t)(BN >> 3) << 17) |
                           ((uint32_t)(TC_BM >> 4) << 24);
    const uint32_t a_lbo = a_mn_major ? TC_BK * 128 : 16, b_lbo = b_mn_major ? TC_BK * 128 : 16;
    const uint32_t a_step = a_mn_major ? 1024 : 32, b_step = b_mn_major ? 1024 : 32;  // per K = 8
    const uint32_t a_sbo = a_mn_major ? 512 : 1024, b_sbo = b_mn_major ? 512 : 1024;
    const uint32_t a_lt = a_mn_major ? 1 : 2, b_lt = b_mn_major ? 1 : 2;
    bool ok = true;
    for (int kb = 0; kb < num_kb && ok; ++kb) {
      const int s = kb % S;
      const uint32_t ph = (kb / S) & 1;
      const int chunk = kb / chunk_kb, buf = chunk & 1;
      const bool chunk_first = (kb % chunk_kb) == 0;
      const bool chunk_last = (kb % chunk_kb) == chunk_kb - 1 || kb == num_kb - 1;
      if (chunk_first) {  // the buffer must have been drained (passes at once for chunks 0 and 1)
        ok = mbar_wait(acc_empty_bar(buf), ((chunk >> 1) & 1) ^ 1, abort_flag);
        if (!ok) break;
      }
      ok = mbar_wait(split_bar(s), ph, abort_flag);
      if (!ok) break;
      tc_fence_after();
      if (lane == 0) {
        const uint32_t d = tmem_d + (uint32_t)(buf * BN);
        const uint32_t d_small = Cfg::SPLIT_ACC ? tmem_d + (uint32_t)(2 * BN + buf * BN) : d;
#pragma unroll
        for (int k = 0; k < TC_BK / 8; ++k) {
          const uint64_t dah = smem_desc(a_hi(s) + k * a_step, a_lbo, a_sbo, a_lt);
          const uint64_t dal = smem_desc(a_lo(s) + k * a_step, a_lbo, a_sbo, a_lt);
          const uint64_t dbh = smem_desc(b_hi(s) + k * b_step, b_lbo, b_sbo, b_lt);
          const uint64_t dbl = smem_desc(b_lo(s) + k * b_step, b_lbo, b_sbo, b_lt);
          const uint32_t fresh = chunk_first && k == 0;             // first MMA of a chunk overwrites
          mma_tf32(d_small, dal, dbh, idesc, !fresh);               // small terms first
          mma_tf32(d_small, dah, dbl, idesc, 1);
          mma_tf32(d, dah, dbh, idesc, Cfg::SPLIT_ACC ? !fresh : 1);
        }
        mma_commit(empty_bar(s));   // frees the stage once these MMAs have read it
        if (chunk_last) mma_commit(acc_full_bar(buf));
      }
      __syncwarp();
    }
    __syncwarp();
  } else if (warp < 6) {
    // ---------------- split transform (and, for 256-wide tiles, half of the drain) ----------------
    const int t = threadIdx.x - 64;  // 0..127
    const int q = warp & 3;
    const uint32_t lane_bits = (uint32_t)(q * 32) << 16;
    const int num_chunks = (num_kb + chunk_kb - 1) / chunk_kb;
    constexpr bool kDrainsToo = Cfg::DRAIN_GROUPS == 2;
    float acc[kDrainsToo ? Cfg::ACC : 1];
#pragma unroll
    for (int j = 0; j < (kDrainsToo ? Cfg::ACC : 1); ++j) acc[j] = 0.f;
    int next_chunk = 0;
    bool ok = true;
    for (int kb = 0; kb < num_kb && ok; ++kb) {
      const int s = kb % S;
      const uint32_t ph = (kb / S) & 1;
      ok = mbar_wait(full_bar(s), ph, abort_flag);
      if (!ok) break;
      float4* ah = reinterpret_cast<float4*>(smem + s * Cfg::STAGE_BYTES);
      float4* al = reinterpret_cast<float4*>(smem + s * Cfg::STAGE_BYTES + Cfg::A_BYTES);
      float4* bh = reinterpret_cast<float4*>(smem + s * Cfg::STAGE_BYTES + 2 * Cfg::A_BYTES);
      float4* bl = reinterpret_cast<float4*>(smem + s * Cfg::STAGE_BYTES + 2 * Cfg::A_BYTES + Cfg::B_BYTES);
      split_tile<Cfg::A_BYTES / 16 / 128>(ah, al, t);
      split_tile<Cfg::B_BYTES / 16 / 128>(bh, bl, t);
      fence_async_smem();   // generic-proxy writes -> visible to the tensor core's async reads
      mbar_arrive(split_bar(s));
      if (kDrainsToo) {
        // drain every chunk that has finished, without waiting for one that has not
        while (next_chunk < num_chunks) {
          const int buf = next_chunk & 1;
          const bool ready = __all_sync(0xffffffffu, mbar_test_wait(acc_full_bar(buf), (next_chunk >> 1) & 1));
          if (!ready) break;
          tc_fence_after();
          drain_add<kDrainsToo ? Cfg::ACC : 32>(tmem_d + lane_bits + (uint32_t)(buf * BN), *reinterpret_cast<float(*)[kDrainsToo ? Cfg::ACC : 32]>(acc));
          tc_fence_before();
          mbar_arrive(acc_empty_bar(buf));
          ++next_chunk;
        }
      }
    }
    if (kDrainsToo) {
      for (; next_chunk < num_chunks && ok; ++next_chunk) {
        const int buf = next_chunk & 1;
        ok = mbar_wait(acc_full_bar(buf), (next_chunk >> 1) & 1, abort_flag);
        __syncwarp();
        if (!ok) break;
        tc_fence_after();
        drain_add<kDrainsToo ? Cfg::ACC : 32>(tmem_d + lane_bits + (uint32_t)(buf * BN), *reinterpret_cast<float(*)[kDrainsToo ? Cfg::ACC : 32]>(acc));
        tc_fence_before();
        mbar_arrive(acc_empty_bar(buf));
      }
      if (ok) {
        // every MMA has completed (last chunk drained): the stage memory is free to stage the tile
        constexpr int NC = kDrainsToo ? Cfg::ACC : 32;
        float* sbuf = reinterpret_cast<float*>(smem) + (warp - 2) * 32 * (NC + 4);
        store_tile<NC>(*reinterpret_cast<float(*)[NC]>(acc), sbuf, c, ldc, m0 + q * 32, n0, M, N, accumulate);
      }
    }
  } else {
    // ---------------- chunk drain, then epilogue ----------------
    const int q = warp & 3;  // TMEM lane quarter this warp may read
    const uint32_t lane_bits = (uint32_t)(q * 32) << 16;
    constexpr int COL0 = (Cfg::DRAIN_GROUPS == 2) ? Cfg::ACC : 0;   // first column of this group
    float acc[Cfg::ACC];
#pragma unroll
    for (int j = 0; j < Cfg::ACC; ++j) acc[j] = 0.f;
    const int num_chunks = (num_kb + chunk_kb - 1) / chunk_kb;
    bool ok = true;
    for (int chunk = 0; chunk < num_chunks && ok; ++chunk) {
      const int buf = chunk & 1;
      ok = mbar_wait(acc_full_bar(buf), (chunk >> 1) & 1, abort_flag);
      __syncwarp();
      if (!ok) break;
      tc_fence_after();
      if (Cfg::SPLIT_ACC) drain_add<Cfg::ACC>(tmem_d + lane_bits + (uint32_t)(2 * BN + buf * BN + COL0), acc);   // small terms first
      drain_add<Cfg::ACC>(tmem_d + lane_bits + (uint32_t)(buf * BN + COL0), acc);
      tc_fence_before();
      mbar_arrive(acc_empty_bar(buf));
    }
    if (ok) {
      // every MMA has completed (last chunk drained): the stage memory is free to stage the tile;
      // with two drain groups the transform warps use the first four slots
      constexpr int SLOT0 = (Cfg::DRAIN_GROUPS == 2) ? 4 : 0;
      float* sbuf = reinterpret_cast<float*>(smem) + (SLOT0 + warp - 6) * 32 * (Cfg::ACC + 4);
      store_tile<Cfg::ACC>(acc, sbuf, c, ldc, m0 + q * 32, n0 + COL0, M, N, accumulate);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_d, Cfg::TMEM_COLS);
  }
  if (threadIdx.x == 0 && *abort_flag && error_flag) *error_flag = 1;
}

// ---- the same GEMM on a pair of SMs --------------------------------------------------
// tcgen05.mma.cta_group::2: two CTAs of a cluster (ranks 0 and 1, consecutive blockIdx.x)
// compute a 256 x 256 tile together.  Each CTA stages its own 128 rows of A and HALF of
// the B tile (128 of the 256 columns); one thread of the rank-0 CTA issues MMAs that read
// both halves and write each CTA's 128 x 256 accumulator rows into that CTA's tensor
// memory.  Per k-block an SM then moves 192 KB through shared memory instead of the 288 KB
// of the 128 x 256 single-CTA tile, which is what bounds that kernel.
//   * tcgen05.alloc / dealloc / commit all carry cta_group::2; warp 1 of BOTH CTAs
//     allocates and frees.
//   * "tiles split" and "accumulator drained" are counted on rank 0's barriers: the
//     peer's warps arrive there remotely (mapa + mbarrier.arrive.shared::cluster).
//   * "stage free" and "chunk ready" exist in both CTAs; rank 0 commits to its own
//     barrier and to the peer's (two plain commits).
//   * Both CTAs meet at a cluster barrier after set-up (the peer's barriers must exist
//     before anyone arrives on them) and before tensor memory is freed.
struct PairConfig {
  static constexpr int A_BYTES = TC_BM * TC_BK * 4;          // this CTA's 128 rows of a
  static constexpr int B_BYTES = 128 * TC_BK * 4;            // this CTA's 128 of the 256 columns of b
  static constexpr int STAGE_BYTES = 2 * (A_BYTES + B_BYTES);
  static constexpr int STAGES = 3;
  static constexpr int BN = 256;
  static constexpr int TMEM_COLS = 512;                      // two accumulator buffers of 256 columns
  static constexpr int ACC = 128;                            // columns per drain group (two groups)
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 + 256;
};

__device__ __forceinline__ void tmem_alloc_pair(uint32_t slot, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(slot), "r"(cols) : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void mma_tf32_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                              uint32_t accumulate) {
  const uint32_t z = 0;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::tf32 [%0], %1, %2, %3, {%5, %5, %5, %5, %5, %5, %5, %5}, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(z)
      : "memory");
}
// bar: a shared::cluster address (this CTA's or the peer's)
__device__ __forceinline__ void mma_commit_pair(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// Arrival on a barrier of this cluster (possibly the other CTA's); what this thread wrote
// before is visible to whoever observes the phase with cluster scope.
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_bar) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_bar) : "memory");
}
// Bounded wait (cluster-scope acquire) on a barrier that threads of both CTAs arrive on.
__device__ __forceinline__ bool mbar_wait_cluster(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
  for (uint32_t it = 0; it < TC_SPIN_LIMIT; ++it) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    if (ok) return true;
    if (it > 64) {
      if (*abort_flag) return false;
      __nanosleep(it > 4096 ? 256 : 32);
    }
  }
  *abort_flag = 1;
  return false;
}
__device__ __forceinline__ uint32_t cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t cluster_addr(uint32_t local_smem_addr, uint32_t cta) {
  uint32_t remote;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local_smem_addr), "r"(cta));
  return remote;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(TC_THREADS, 1)
gemm_tf32x3_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                        float* __restrict__ c, int M, int N, int K, int64_t ldc, int accumulate,
                        int a_mn_major, int b_mn_major, int* error_flag, int kb_per_split,
                        int64_t split_stride) {
  using Cfg = PairConfig;
  constexpr int S = Cfg::STAGES;
  constexpr int BN = Cfg::BN;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + S * Cfg::STAGE_BYTES);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 3 * S + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_rank();          // 0 issues the MMAs
  const bool leader = rank == 0;
  const int m0 = blockIdx.x * TC_BM;             // this CTA's rows (the pair: blockIdx.x = 2p, 2p + 1)
  const int n0 = blockIdx.y * BN;                // the pair's columns; this CTA stages [n0 + 128 rank, + 128)
  const int nb0 = n0 + 128 * (int)rank;
  const int kb_begin = blockIdx.z * kb_per_split;
  const int num_kb = min((K + TC_BK - 1) / TC_BK - kb_begin, kb_per_split);
  c += (int64_t)blockIdx.z * split_stride;
  const uint32_t bar0 = smem_u32(bars);
  auto full_bar = [&](int s) { return bar0 + 8u * s; };
  auto split_bar = [&](int s) { return bar0 + 8u * (S + s); };
  auto empty_bar = [&](int s) { return bar0 + 8u * (2 * S + s); };
  auto acc_full_bar = [&](int b) { return bar0 + 8u * (3 * S + b); };
  auto acc_empty_bar = [&](int b) { return bar0 + 8u * (3 * S + 2 + b); };
  const uint32_t smem_base = smem_u32(smem);
  auto a_hi = [&](int s) { return smem_base + s * Cfg::STAGE_BYTES; };
  auto a_lo = [&](int s) { return a_hi(s) + Cfg::A_BYTES; };
  auto b_hi = [&](int s) { return a_hi(s) + 2 * Cfg::A_BYTES; };
  auto b_lo = [&](int s) { return b_hi(s) + Cfg::B_BYTES; };
  // rank 0's copies of the two barriers that count arrivals from both CTAs
  auto lead_split_bar = [&](int s) { return cluster_addr(split_bar(s), 0); };
  auto lead_acc_empty_bar = [&](int b) { return cluster_addr(acc_empty_bar(b), 0); };

  if (threadIdx.x == 0) {
    for (int s = 0; s < S; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(split_bar(s), 256);      // the transform threads of both CTAs
      mbar_init(empty_bar(s), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(acc_full_bar(b), 1);
      mbar_init(acc_empty_bar(b), 512);  // both drain groups of both CTAs
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  pdl_launch_dependents();
  if (warp == 0 && lane == 0) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_a) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_b) : "memory");
  }
  if (warp == 1) tmem_alloc_pair(smem_u32(tmem_slot), Cfg::TMEM_COLS);
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();        // both CTAs: barriers initialised, tensor memory allocated
  tc_fence_after();
  const uint32_t tmem_d = *tmem_slot;
  pdl_wait();

  if (warp == 0) {
    // ---------------- TMA producer (this CTA's tiles) ----------------
    if (lane == 0) {
      int issued = 0;
      for (int kb = 0; kb < num_kb; ++kb) {
        const int s = kb % S;
        const uint32_t ph = (kb / S) & 1;
        if (!mbar_wait(empty_bar(s), ph ^ 1, abort_flag)) break;
        mbar_expect_tx(full_bar(s), Cfg::A_BYTES + Cfg::B_BYTES);
        const int k0 = (kb_begin + kb) * TC_BK;
        if (!a_mn_major) {
          tma_load_2d(a_hi(s), &map_a, k0, m0, full_bar(s));
        } else {
#pragma unroll
          for (int j = 0; j < TC_BM / 32; ++j)
            tma_load_2d(a_hi(s) + j * (TC_BK * 128), &map_a, m0 + 32 * j, k0, full_bar(s));
        }
        if (!b_mn_major) {
          tma_load_2d(b_hi(s), &map_b, k0, nb0, full_bar(s));
        } else {
#pragma unroll
          for (int j = 0; j < 128 / 32; ++j)
            tma_load_2d(b_hi(s) + j * (TC_BK * 128), &map_b, nb0 + 32 * j, k0, full_bar(s));
        }
        issued = kb + 1;
      }
      if (*abort_flag) {
        const int first = issued > S ? issued - S : 0;
        for (int kb = first; kb < issued; ++kb) {
          const uint32_t bar = full_bar(kb % S), ph = (kb / S) & 1;
          for (uint32_t it = 0; it < TC_SPIN_LIMIT && !mbar_try_wait(bar, ph); ++it) __nanosleep(64);
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ---------------- MMA issuer: rank 0 only ----------------
    if (leader) {
      const uint32_t idesc = (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(a_mn_major != 0) << 15) |
                             ((uint32_t)(b_mn_major != 0) << 16) | ((uint32_t)(BN >> 3) << 17) |
                             ((uint32_t)((2 * TC_BM) >> 4) << 24);
      const uint32_t a_lbo = a_mn_major ? TC_BK * 128 : 16, b_lbo = b_mn_major ? TC_BK * 128 : 16;
      const uint32_t a_step = a_mn_major ? 1024 : 32, b_step = b_mn_major ? 1024 : 32;
      const uint32_t a_sbo = a_mn_major ? 512 : 1024, b_sbo = b_mn_major ? 512 : 1024;
      const uint32_t a_lt = a_mn_major ? 1 : 2, b_lt = b_mn_major ? 1 : 2;
      bool ok = true;
      for (int kb = 0; kb < num_kb && ok; ++kb) {
        const int s = kb % S;
        const uint32_t ph = (kb / S) & 1;
        const int chunk = kb / TC_CHUNK_KB, buf = chunk & 1;
        const bool chunk_first = (kb % TC_CHUNK_KB) == 0;
        const bool chunk_last = (kb % TC_CHUNK_KB) == TC_CHUNK_KB - 1 || kb == num_kb - 1;
        if (chunk_first) {
          ok = mbar_wait_cluster(acc_empty_bar(buf), ((chunk >> 1) & 1) ^ 1, abort_flag);
          if (!ok) break;
        }
        ok = mbar_wait_cluster(split_bar(s), ph, abort_flag);   // both CTAs' tiles are split
        if (!ok) break;
        tc_fence_after();
        if (lane == 0) {
          const uint32_t d = tmem_d + (uint32_t)(buf * BN);
#pragma unroll
          for (int k = 0; k < TC_BK / 8; ++k) {
            const uint64_t dah = smem_desc(a_hi(s) + k * a_step, a_lbo, a_sbo, a_lt);
            const uint64_t dal = smem_desc(a_lo(s) + k * a_step, a_lbo, a_sbo, a_lt);
            const uint64_t dbh = smem_desc(b_hi(s) + k * b_step, b_lbo, b_sbo, b_lt);
            const uint64_t dbl = smem_desc(b_lo(s) + k * b_step, b_lbo, b_sbo, b_lt);
            mma_tf32_pair(d, dal, dbh, idesc, !(chunk_first && k == 0));
            mma_tf32_pair(d, dah, dbl, idesc, 1);
            mma_tf32_pair(d, dah, dbh, idesc, 1);
          }
          mma_commit_pair(empty_bar(s));                       // this CTA's stage ...
          mma_commit_pair(cluster_addr(empty_bar(s), 1));      // ... and the peer's
          if (chunk_last) {
            mma_commit_pair(acc_full_bar(buf));
            mma_commit_pair(cluster_addr(acc_full_bar(buf), 1));
          }
        }
        __syncwarp();
      }
    }
    __syncwarp();
  } else if (warp < 6) {
    // ---------------- split transform + drain of columns [0, 128) ----------------
    const int t = threadIdx.x - 64;
    const int q = warp & 3;
    const uint32_t lane_bits = (uint32_t)(q * 32) << 16;
    const int num_chunks = (num_kb + TC_CHUNK_KB - 1) / TC_CHUNK_KB;
    float acc[Cfg::ACC];
#pragma unroll
    for (int j = 0; j < Cfg::ACC; ++j) acc[j] = 0.f;
    int next_chunk = 0;
    bool ok = true;
    auto drain = [&](int chunk_idx) {
      const int buf = chunk_idx & 1;
      tc_fence_after();
      drain_add<Cfg::ACC>(tmem_d + lane_bits + (uint32_t)(buf * BN), acc);
      tc_fence_before();
      mbar_arrive_cluster(lead_acc_empty_bar(buf));
    };
    for (int kb = 0; kb < num_kb && ok; ++kb) {
      const int s = kb % S;
      const uint32_t ph = (kb / S) & 1;
      ok = mbar_wait(full_bar(s), ph, abort_flag);
      if (!ok) break;
      float4* ah = reinterpret_cast<float4*>(smem + s * Cfg::STAGE_BYTES);
      float4* al = reinterpret_cast<float4*>(smem + s * Cfg::STAGE_BYTES + Cfg::A_BYTES);
      float4* bh = reinterpret_cast<float4*>(smem + s * Cfg::STAGE_BYTES + 2 * Cfg::A_BYTES);
      float4* bl = reinterpret_cast<float4*>(smem + s * Cfg::STAGE_BYTES + 2 * Cfg::A_BYTES + Cfg::B_BYTES);
      split_tile<Cfg::A_BYTES / 16 / 128>(ah, al, t);
      split_tile<Cfg::B_BYTES / 16 / 128>(bh, bl, t);
      fence_async_smem();
      mbar_arrive_cluster(lead_split_bar(s));
      while (next_chunk < num_chunks) {   // drain what has finished, never wait for what has not
        const bool ready = __all_sync(0xffffffffu, mbar_test_wait(acc_full_bar(next_chunk & 1), (next_chunk >> 1) & 1));
        if (!ready) break;
        drain(next_chunk);
        ++next_chunk;
      }
    }
    for (; next_chunk < num_chunks && ok; ++next_chunk) {
      ok = mbar_wait(acc_full_bar(next_chunk & 1), (next_chunk >> 1) & 1, abort_flag);
      __syncwarp();
      if (!ok) break;
      drain(next_chunk);
    }
    if (ok) {
      float* sbuf = reinterpret_cast<float*>(smem) + (warp - 2) * 32 * (Cfg::ACC + 4);
      store_tile<Cfg::ACC>(acc, sbuf, c, ldc, m0 + q * 32, n0, M, N, accumulate);
    }
  } else {
    // ---------------- drain of columns [128, 256), then epilogue ----------------
    const int q = warp & 3;
    const uint32_t lane_bits = (uint32_t)(q * 32) << 16;
    float acc[Cfg::ACC];
#pragma unroll
    for (int j = 0; j < Cfg::ACC; ++j) acc[j] = 0.f;
    const int num_chunks = (num_kb + TC_CHUNK_KB - 1) / TC_CHUNK_KB;
    bool ok = true;
    for (int chunk = 0; chunk < num_chunks && ok; ++chunk) {
      const int buf = chunk & 1;
      ok = mbar_wait(acc_full_bar(buf), (chunk >> 1) & 1, abort_flag);
      __syncwarp();
      if (!ok) break;
      tc_fence_after();
      drain_add<Cfg::ACC>(tmem_d + lane_bits + (uint32_t)(buf * BN + Cfg::ACC), acc);
      tc_fence_before();
      mbar_arrive_cluster(lead_acc_empty_bar(buf));
    }
    if (ok) {
      float* sbuf = reinterpret_cast<float*>(smem) + (4 + warp - 6) * 32 * (Cfg::ACC + 4);
      store_tile<Cfg::ACC>(acc, sbuf, c, ldc, m0 + q * 32, n0 + Cfg::ACC, M, N, accumulate);
    }
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();        // nobody in the pair reads shared or tensor memory of the other any more
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_d, Cfg::TMEM_COLS);
  }
  if (threadIdx.x == 0 && *abort_flag && error_flag) *error_flag = 1;
}

// out[m, n] (+)= sum over splits of partial[s][m][n], splits added in index order.
__global__ void __launch_bounds__(256)
splitk_reduce_kernel(const float* __restrict__ partial, int splits, int64_t split_stride, float* out,
                     int64_t M, int64_t N, int64_t ldp, int64_t ldc, int accumulate) {
  const int64_t groups_per_row = ldp >> 2;
  const int64_t total = M * groups_per_row;
  const bool vec_out = ((reinterpret_cast<uintptr_t>(out) & 15) == 0) && (ldc % 4 == 0);
  for (int64_t g = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; g < total;
       g += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = g / groups_per_row, c0 = (g - r * groups_per_row) << 2;
    float4 acc = *reinterpret_cast<const float4*>(partial + r * ldp + c0);
    for (int s = 1; s < splits; ++s) {
      const float4 v = *reinterpret_cast<const float4*>(partial + (int64_t)s * split_stride + r * ldp + c0);
      acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
    }
    float* o = out + r * ldc + c0;
    if (vec_out && c0 + 4 <= N) {
      if (accumulate) {
        const float4 old = *reinterpret_cast<const float4*>(o);
        acc.x += old.x; acc.y += old.y; acc.z += old.z; acc.w += old.w;
      }
      *reinterpret_cast<float4*>(o) = acc;
    } else {
      const float v[4] = {acc.x, acc.y, acc.z, acc.w};
      for (int j = 0; j < 4; ++j)
        if (c0 + j < N) o[j] = accumulate ? o[j] + v[j] : v[j];
    }
  }
}

// Copy of a row-pitched matrix whose base or pitch TMA cannot address (base not on a
// 16-byte boundary, pitch not a multiple of 4 floats) into an aligned, padded
// temporary: dst row pitch ldd is a multiple of 4, the pad columns are zero.
__global__ void __launch_bounds__(256)
stage_operand_kernel(const float* __restrict__ src, int64_t rows, int64_t cols, int64_t lds,
                     float* __restrict__ dst, int64_t ldd) {
  const int64_t groups_per_row = ldd >> 2;
  const int64_t total = rows * groups_per_row;
  for (int64_t g = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; g < total;
       g += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = g / groups_per_row, c = (g - r * groups_per_row) << 2;
    const float* p = src + r * lds + c;
    float4 v;
    v.x = (c < cols) ? p[0] : 0.f;
    v.y = (c + 1 < cols) ? p[1] : 0.f;
    v.z = (c + 2 < cols) ? p[2] : 0.f;
    v.w = (c + 3 < cols) ? p[3] : 0.f;
    *reinterpret_cast<float4*>(dst + r * ldd + c) = v;
  }
}

// ---- host side ---------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);

struct TcHost {
  EncodeTiledFn encode = nullptr;
  int* error_flag_host = nullptr;   // mapped pinned memory
  int* error_flag_dev = nullptr;
  // split-K partial tiles (stream-ordered allocation), one buffer per compute stream:
  // GEMMs of the two streams may run at the same time
  float* partial[2] = {nullptr, nullptr};
  size_t partial_bytes[2] = {0, 0};
  std::mutex mu;
  struct Key {
    const void* p; int64_t inner, outer, ld; int box_outer; int mn_major;
    bool operator==(const Key& o) const {
      return p == o.p && inner == o.inner && outer == o.outer && ld == o.ld && box_outer == o.box_outer &&
             mn_major == o.mn_major;
    }
  };
  struct KeyHash {
    size_t operator()(const Key& k) const {
      size_t h = (size_t)k.p;
      h ^= (size_t)k.inner * 0x9E3779B97F4A7C15ull + (h << 6);
      h ^= (size_t)k.outer * 0xC2B2AE3D27D4EB4Full + (h >> 3);
      h ^= (size_t)k.ld * 0x165667B19E3779F9ull + (size_t)k.box_outer * 2 + (size_t)k.mn_major;
      return h;
    }
  };
  std::unordered_map<Key, CUtensorMap, KeyHash> cache;
};
static TcHost& tc_host() {
  static TcHost h;
  return h;
}

static int tc_setup() {
  TcHost& h = tc_host();
  if (h.encode) return B200_OK;
  void* fn = nullptr;
  cudaDriverEntryPointQueryResult q;
  B200_CUDA(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q));
  B200_REQUIRE(fn != nullptr && q == cudaDriverEntryPointSuccess, "cuTensorMapEncodeTiled is unavailable");
  B200_CUDA(cudaHostAlloc((void**)&h.error_flag_host, sizeof(int), cudaHostAllocMapped));
  *h.error_flag_host = 0;
  B200_CUDA(cudaHostGetDevicePointer((void**)&h.error_flag_dev, h.error_flag_host, 0));
  B200_CUDA(cudaFuncSetAttribute(gemm_tf32x3_kernel<32>, cudaFuncAttributeMaxDynamicSharedMemorySize, TcConfig<32>::SMEM_BYTES));
  B200_CUDA(cudaFuncSetAttribute(gemm_tf32x3_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, TcConfig<64>::SMEM_BYTES));
  B200_CUDA(cudaFuncSetAttribute(gemm_tf32x3_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, TcConfig<128>::SMEM_BYTES));
  B200_CUDA(cudaFuncSetAttribute(gemm_tf32x3_kernel<256>, cudaFuncAttributeMaxDynamicSharedMemorySize, TcConfig<256>::SMEM_BYTES));
  B200_CUDA(cudaFuncSetAttribute(gemm_tf32x3_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, PairConfig::SMEM_BYTES));
  h.encode = (EncodeTiledFn)fn;
  return B200_OK;
}

// 2-D fp32 tensor map over a row-major array: `outer` rows of `inner` contiguous
// elements, row pitch ld; box = 32 x box_outer, zero fill, 128-byte swizzle in the
// flavour the operand's major-ness needs.
static int tc_map(const float* p, int64_t inner, int64_t outer, int64_t ld, int box_outer, int mn_major,
                  CUtensorMap* out) {
  TcHost& h = tc_host();
  TcHost::Key key{p, inner, outer, ld, box_outer, mn_major};
  auto it = h.cache.find(key);
  if (it != h.cache.end()) {
    *out = it->second;
    return B200_OK;
  }
  cuuint64_t dims[2] = {(cuuint64_t)inner, (cuuint64_t)outer};
  cuuint64_t strides[1] = {(cuuint64_t)ld * 4};
  cuuint32_t box[2] = {32u, (cuuint32_t)box_outer};
  cuuint32_t estr[2] = {1u, 1u};
  CUresult r = h.encode(out, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, (void*)p, dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE,
                        mn_major ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : CU_TENSOR_MAP_SWIZZLE_128B,
                        CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return set_error(B200_ERR_CUDA, "cuTensorMapEncodeTiled failed with %d", (int)r);
  if (h.cache.size() > 8192) h.cache.clear();
  h.cache.emplace(key, *out);
  return B200_OK;
}

// The device-visible word that kernels with bounded waits raise when they give up
// (mapped host memory; NULL if it cannot be set up).
int* device_error_flag() {
  std::lock_guard<std::mutex> lock(tc_host().mu);
  if (tc_setup() != B200_OK) return nullptr;
  return tc_host().error_flag_dev;
}

// Reports (and clears) a timeout raised by a kernel (a tensor-core GEMM waiting on a
// barrier, a peer all-reduce waiting for another rank).  Called by the synchronising
// entry points after the stream has drained.
void peer_disable();   // peer.cu

int gemm_tc_check_flag() {
  TcHost& h = tc_host();
  if (h.error_flag_host && *h.error_flag_host) {
    *h.error_flag_host = 0;
    peer_disable();
    return set_error(B200_ERR_DEVICE_FLAG,
                     "a kernel gave up waiting (a tensor-core GEMM on a barrier, or a peer all-reduce on another "
                     "rank); its output is invalid");
  }
  return B200_OK;
}

// Views handed out by the reference's memory layer start at arbitrary element
// offsets of one flat buffer, so most operands are NOT on a 16-byte boundary.  Such
// an operand (or one whose pitch is not a multiple of 4 floats, e.g. 205 columns) is
// first copied into an aligned stream-ordered temporary; the copy moves 8 bytes per
// element against the 2*N (or 2*M) flops per element of the GEMM that follows.
struct Staged {
  const float* ptr = nullptr;
  int64_t ld = 0;
  float* temp = nullptr;
};
static int stage_if_needed(const float* p, int64_t rows, int64_t cols, int64_t ld, Staged* out) {
  out->ptr = p;
  out->ld = ld;
  out->temp = nullptr;
  if (aligned16(p) && ld % 4 == 0) return B200_OK;
  const State& s = state();
  const int64_t ldd = (cols + 3) & ~(int64_t)3;
  B200_CUDA(cudaMallocAsync((void**)&out->temp, (size_t)rows * ldd * sizeof(float), s.stream));
  int64_t blocks = ceil_div(rows * (ldd >> 2), 256);
  if (blocks > (int64_t)s.sm_count * 16) blocks = (int64_t)s.sm_count * 16;
  stage_operand_kernel<<<(unsigned)blocks, 256, 0, s.stream>>>(p, rows, cols, ld, out->temp, ldd);
  B200_LAUNCH_CHECK();
  out->ptr = out->temp;
  out->ld = ldd;
  return B200_OK;
}
static void release(Staged* st) {
  if (st->temp) cudaFreeAsync(st->temp, state().stream);
  st->temp = nullptr;
}

// Where a GEMM left its result when the caller asked to finish split-K itself:
// `splits` partial matrices of pitch ld, split_stride floats apart, to be added in
// index order.  The buffer belongs to the library and is valid until the next GEMM
// on the stream.
struct GemmPartials {
  const float* ptr;
  int splits;
  int64_t split_stride;
  int64_t ld;
};

// k-blocks accumulated in tensor memory between two drains (b200_set_tuning key 9).  Every
// tcgen05.mma adds into its fp32 accumulator with truncation toward zero; with operands of
// one sign the result of a chunk of c k-blocks comes out smaller by about c * 6.5e-7 of
// itself (measured: 5.3e-6 / 2.6e-6 / 1.3e-6 / 7e-7 for c = 8 / 4 / 2 / 1, at 220 / 219 / 216 /
// 209 TFLOP/s for 8192 x 4096 x 4096).  Two k-blocks (64 along K) is the default.
static inline int chunk_k_blocks(const State& s) {
  return (s.gemm_chunk_kb == 1 || s.gemm_chunk_kb == 2 || s.gemm_chunk_kb == 4 || s.gemm_chunk_kb == 8) ? s.gemm_chunk_kb : 2;
}

static int gemm_tc_impl(int transa, int transb, int64_t M, int64_t N, int64_t K, const float* a, int64_t lda,
                        const float* b, int64_t ldb, float* c, int64_t ldc, int accumulate,
                        GemmPartials* partials_out) {
  std::lock_guard<std::mutex> lock(tc_host().mu);
  if (int rc = tc_setup()) return rc;
  const State& s = state();
  Staged sa, sb;
  if (int rc = stage_if_needed(a, transa ? K : M, transa ? M : K, lda, &sa)) return rc;
  if (int rc = stage_if_needed(b, transb ? N : K, transb ? K : N, ldb, &sb)) { release(&sa); return rc; }
  a = sa.ptr; lda = sa.ld;
  b = sb.ptr; ldb = sb.ld;
  // Tile width.  One tcgen05.mma costs about the same time for any N <= 128 (it is
  // bound by streaming the 128-row A operand) and under twice that for N = 256, so
  // the tile is as wide as N allows; 256 only while its tiles still fill the GPU.
  const int64_t tiles_m = ceil_div(M, TC_BM);
  int bn = N <= 32 ? 32 : (N <= 64 ? 64 : 128);
  if (N >= 256 && 2 * tiles_m * ceil_div(N, 256) >= s.sm_count) bn = 256;
  if (s.gemm_bn == 32 || s.gemm_bn == 64 || s.gemm_bn == 128 || s.gemm_bn == 256) bn = s.gemm_bn;
  const int64_t tiles = tiles_m * ceil_div(N, bn);
  // Split-K when the tiles alone cannot fill the GPU: every CTA then walks a short
  // K range (a multiple of the TMEM chunk) and writes a partial tile; a second
  // kernel adds the partials in a fixed order.
  const int total_kb = (int)ceil_div(K, TC_BK);
  // tiles of up to 128 columns keep the small terms in their own accumulator and can afford twice the chunk
  const int chunk_kb = (bn <= 128 && s.gemm_chunk_kb == 0) ? 4 : chunk_k_blocks(s);
  int splits = 1, kb_per_split = total_kb;
  const int64_t sms = s.sm_count / s.sm_share;
  const int chunk_unit = chunk_kb > TC_CHUNK_KB ? chunk_kb : TC_CHUNK_KB;   // a split is a whole number of chunks (pair kernel: its own)
  if (tiles * 2 <= sms && total_kb >= 2 * chunk_unit) {
    int want = (int)(sms / tiles);
    kb_per_split = (int)ceil_div(total_kb, want);
    kb_per_split = (int)ceil_div(kb_per_split, chunk_unit) * chunk_unit;
    splits = (int)ceil_div(total_kb, kb_per_split);
  }
  float* dst = c;
  int64_t dst_ld = ldc, split_stride = 0;
  int acc_flag = accumulate;
  if (splits > 1) {
    dst_ld = (N + 3) & ~(int64_t)3;
    split_stride = M * dst_ld;
    const size_t need = (size_t)splits * split_stride * sizeof(float);
    TcHost& h = tc_host();
    const int si = s.stream_index;
    if (h.partial_bytes[si] < need) {
      // the buffer outlives the call, so it must not become an allocation of a recorded graph
      B200_REQUIRE(!s.capturing, "the split-K work buffer would have to grow while a graph is being recorded: "
                                 "run the step once before recording it");
      retire_work_buffer(h.partial[si]);   // a recorded graph may still replay into the old buffer
      h.partial[si] = nullptr;
      h.partial_bytes[si] = 0;
      B200_CUDA(cudaMallocAsync((void**)&h.partial[si], need, s.stream));
      h.partial_bytes[si] = need;
    }
    dst = h.partial[si];
    acc_flag = 0;
  }
  CUtensorMap ma, mb;
  // A: K-major when not transposed (array is M x K), MN-major when transposed (K x M)
  if (int rc = transa ? tc_map(a, M, K, lda, TC_BK, 1, &ma) : tc_map(a, K, M, lda, TC_BM, 0, &ma)) { release(&sa); release(&sb); return rc; }
  // B: K-major when transposed (array is N x K), MN-major when not (K x N)
  if (int rc = transb ? tc_map(b, K, N, ldb, bn, 0, &mb) : tc_map(b, N, K, ldb, TC_BK, 1, &mb)) { release(&sa); release(&sb); return rc; }
  dim3 grid((unsigned)ceil_div(N, bn), (unsigned)tiles_m, (unsigned)splits);
  const bool pair = bn == 256 && s.gemm_pair;
  if (pair)   // CTA pairs along x = M (rows past M are zero-filled and not stored), column tiles along y
    grid = dim3((unsigned)(ceil_div(tiles_m, 2) * 2), (unsigned)ceil_div(N, bn), (unsigned)splits);
  int* flag = tc_host().error_flag_dev;
  const int m = (int)M, n = (int)N, k = (int)K;
  const int amn = transa ? 1 : 0, bmn = transb ? 0 : 1;
  if (pair) {
    CUtensorMap mbh;   // the pair's b tile arrives as two halves of 128 columns, one per CTA
    if (int rc = transb ? tc_map(b, K, N, ldb, 128, 0, &mbh) : tc_map(b, N, K, ldb, TC_BK, 1, &mbh)) { release(&sa); release(&sb); return rc; }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(TC_THREADS);
    cfg.dynamicSmemBytes = PairConfig::SMEM_BYTES;
    cfg.stream = s.stream;
    cudaLaunchAttribute attr[1];     // the cluster shape (2 x 1 x 1) is part of the kernel's declaration
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = s.pdl_now ? 1 : 0;
    const cudaError_t le = cudaLaunchKernelEx(&cfg, gemm_tf32x3_pair_kernel, ma, mbh, dst, m, n, k, dst_ld, acc_flag, amn,
                                              bmn, flag, kb_per_split, split_stride);
    if (le != cudaSuccess) {
      int clusters = -1;
      cudaOccupancyMaxActiveClusters(&clusters, gemm_tf32x3_pair_kernel, &cfg);
      cudaGetLastError();
      release(&sa); release(&sb);
      return set_error(B200_ERR_CUDA, "pair GEMM launch failed: %s (grid %u x %u x %u, cluster 2 x 1 x 1, %d bytes of "
                       "shared memory, %d clusters can be resident)", cudaGetErrorString(le), grid.x, grid.y, grid.z,
                       (int)PairConfig::SMEM_BYTES, clusters);
    }
  } else switch (bn) {
    case 32: B200_CUDA(launch_maybe_pdl(s.pdl_now, gemm_tf32x3_kernel<32>, grid, dim3(TC_THREADS), (size_t)TcConfig<32>::SMEM_BYTES, s.stream, ma, mb, dst, m, n, k, dst_ld, acc_flag, amn, bmn, flag, kb_per_split, split_stride, chunk_kb)); break;
    case 64: B200_CUDA(launch_maybe_pdl(s.pdl_now, gemm_tf32x3_kernel<64>, grid, dim3(TC_THREADS), (size_t)TcConfig<64>::SMEM_BYTES, s.stream, ma, mb, dst, m, n, k, dst_ld, acc_flag, amn, bmn, flag, kb_per_split, split_stride, chunk_kb)); break;
    case 256: B200_CUDA(launch_maybe_pdl(s.pdl_now, gemm_tf32x3_kernel<256>, grid, dim3(TC_THREADS), (size_t)TcConfig<256>::SMEM_BYTES, s.stream, ma, mb, dst, m, n, k, dst_ld, acc_flag, amn, bmn, flag, kb_per_split, split_stride, chunk_kb)); break;
    default: B200_CUDA(launch_maybe_pdl(s.pdl_now, gemm_tf32x3_kernel<128>, grid, dim3(TC_THREADS), (size_t)TcConfig<128>::SMEM_BYTES, s.stream, ma, mb, dst, m, n, k, dst_ld, acc_flag, amn, bmn, flag, kb_per_split, split_stride, chunk_kb)); break;
  }
  B200_LAUNCH_CHECK();
  if (partials_out) {
    partials_out->ptr = dst;
    partials_out->splits = splits;
    partials_out->split_stride = split_stride;
    partials_out->ld = dst_ld;
  } else if (splits > 1) {
    const int64_t total = M * dst_ld;
    int64_t blocks = ceil_div(total / 4, 256);
    if (blocks > (int64_t)s.sm_count * 8) blocks = (int64_t)s.sm_count * 8;
    splitk_reduce_kernel<<<(unsigned)blocks, 256, 0, s.stream>>>(dst, splits, split_stride, c, M, N, dst_ld, ldc, accumulate);
    B200_LAUNCH_CHECK();
  }
  release(&sa);
  release(&sb);
  return B200_OK;
}

int gemm_tc(int transa, int transb, int64_t M, int64_t N, int64_t K, const float* a, int64_t lda,
            const float* b, int64_t ldb, float* c, int64_t ldc, int accumulate) {
  // tiny problems: the CUDA-core kernel has less fixed cost
  if (M * N * K < (int64_t)64 * 64 * 64 && state().gemm_path != 2) return B200_ERR_UNSUPPORTED;
  return gemm_tc_impl(transa, transb, M, N, K, a, lda, b, ldb, c, ldc, accumulate, nullptr);
}

// out = op(a).op(b) into `c` (pitch ldc) when one pass suffices, or into the library's
// partial buffer when the problem was split along K; *where says which.
int gemm_tc_partials(int transa, int transb, int64_t M, int64_t N, int64_t K, const float* a, int64_t lda,
                     const float* b, int64_t ldb, float* c, int64_t ldc, const float** ptr, int* splits,
                     int64_t* split_stride, int64_t* ld) {
  GemmPartials p;
  if (int rc = gemm_tc_impl(transa, transb, M, N, K, a, lda, b, ldb, c, ldc, 0, &p)) return rc;
  *ptr = p.ptr;
  *splits = p.splits;
  *split_stride = p.split_stride;
  *ld = p.ld;
  return B200_OK;
}

}  // namespace b200
