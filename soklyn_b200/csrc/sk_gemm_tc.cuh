// Tensor-core GEMM for the 16-bit DenseBlock path on sm_100a.
//
//   C[M x N] = A . B, f16 or bf16 operands, f32 accumulation in tensor memory (TMEM).
//
// One persistent CTA per SM walks output tiles of 128 x BN. Warp 0 streams operand panels
// (64 deep in K) from global memory into a ring of shared-memory stages with TMA tile loads
// (128-byte swizzle); one thread of warp 1 issues tcgen05.mma instructions (M=128, N=BN, K=16)
// that read the stages through shared-memory descriptors and accumulate into one of two TMEM
// accumulator buffers; eight epilogue warps drain the other buffer with tcgen05.ld, pass each
// 32 x 32 block through shared memory so that global accesses run along rows, and apply the
// fused epilogue functor (sk_epilogue.cuh). Mainloop and epilogue of consecutive tiles overlap.
//
// Both operand layouts come straight from the row-major tensors, no transposed copies:
//   K-major  operand: element (mn, k) at ptr[mn * ld + k]  -> one TMA box {64 k, rows}
//   MN-major operand: element (mn, k) at ptr[k * ld + mn]  -> boxes {64 mn, 64 k}, 8 KiB apart
// so forward (X K-major, W MN-major), dX (dY, W both K-major) and dW (X, dY both MN-major)
// use the same kernel. Out-of-range parts of a box are zero-filled by TMA; the epilogue
// clips rows and columns.
//
// f32 operands (SPLIT = true): each f32 matrix is split beforehand into three bf16 matrices a0 + a1 + a2
// (8 significant bits each, 24 together), and the product is accumulated from the six partial products
// whose weight is at least 2^-16 of the leading one, smallest first: a2.b0, a0.b2, a1.b1, a1.b0, a0.b1,
// a0.b0. For every 64-deep K step the producer loads the six part tiles once and the MMA thread multiplies
// the six pairs in turn; the sum over K is finished in registers (see TcSplitMaps); everything else is the
// 16-bit kernel. Every barrier wait is bounded; on a timeout the kernel records an
// error code and leaves.
#pragma once

#include <type_traits>

#include "sk_epilogue.cuh"
#include "sk_tc_ptx.cuh"

namespace sk {

constexpr int kTcBM = 128;          // tile rows = UMMA M
constexpr int kTcBK = 64;           // K depth of one stage: 64 x 2 B = one 128-byte swizzle row
constexpr int kTcEpiWarps = 8;
constexpr int kTcThreads = (2 + kTcEpiWarps) * 32;
constexpr int kTcABytes = kTcBM * kTcBK * 2;

template <int BN> struct TcShape {
    static constexpr int kBBytes = BN * kTcBK * 2;
    static constexpr int kStageBytes = kTcABytes + kBBytes;
    static constexpr int kStages = BN == 256 ? 4 : 6;
    static constexpr int kTmemCols = 2 * BN;                       // two accumulator buffers
    static constexpr int kEpiBufBytes = kTcEpiWarps * 32 * 33 * 4;
    static constexpr int kBarBytes = (2 * kStages + 4) * 8 + 16;
    static constexpr int kSmemBytes = 1024 /*alignment slack*/ + kStages * kStageBytes + kEpiBufBytes + kBarBytes;
};

// Passes of the epilogue whose loads are in flight together: functors may declare kGroup (1, 2 or 4).
template <class Epi, class = void> struct EpiGroup { static constexpr int value = 1; };
template <class Epi> struct EpiGroup<Epi, decltype((void)Epi::kGroup)> { static constexpr int value = Epi::kGroup; };
// Functors that keep running sums over the passes of a chunk declare kHasAcc, Acc, acc_init, acc_flush
// and take the accumulator as the last argument of finish().
template <class Epi, class = void> struct EpiAcc { static constexpr bool value = false; struct type {}; };
template <class Epi> struct EpiAcc<Epi, std::enable_if_t<Epi::kHasAcc>> { static constexpr bool value = true; using type = typename Epi::Acc; };
// Functors whose body is small enough to exist four times declare kPingPong = true.
template <class Epi, class = void> struct EpiPingPong { static constexpr bool value = false; };
template <class Epi> struct EpiPingPong<Epi, decltype((void)Epi::kPingPong)> { static constexpr bool value = Epi::kPingPong; };

enum : int { kTcErrProducer = 1, kTcErrMma = 2, kTcErrEpilogue = 3, kTcErrGate = 4 };

// Optional gate on the B operand (data-parallel backward): the rows of B arrive from other GPUs in
// `chunks` blocks of `rows_per_chunk` rows, and flags[chunk * stride + rank] reaches `epoch` once that
// rank's part of the block has landed in this GPU's memory (this GPU's own part is complete before the
// launch, by stream order). The producer waits (bounded) for every rank's
// flag of the blocks a tile needs before it issues the loads. flags == nullptr: no gate.
struct TcGate {
    const uint32_t *flags;
    uint32_t world, self, stride, chunks, rows_per_chunk, epoch;   // `self`: the rank whose rows are ordered by the stream
};

// Bounded wait until *flag (system-scope acquire) has reached `value` in wrap-around order.
__device__ __forceinline__ bool wait_flag_reached(const uint32_t *flag, uint32_t value) {
    const long long t0 = clock64();
    for (;;) {
        uint32_t v;
        asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
        if ((int32_t)(v - value) >= 0) return true;
        if (clock64() - t0 > 4000000000LL) return false;
        __nanosleep(100);
    }
}

// Tile order. Tiles are walked in groups of group_n tile-columns (8 by default), row-major inside a group, so
// that the ~148 tiles in flight form a compact block (about 18 x 8 tiles): the B panels of a group
// stay in L2 while A streams past once per group, instead of once per tile-column.
__device__ __forceinline__ void tile_coords(uint32_t tile, uint32_t tiles_m, uint32_t tiles_n, uint32_t group_n,
                                            uint32_t &mi, uint32_t &ni) {
    const uint32_t group_tiles = group_n * tiles_m;
    const uint32_t g = tile / group_tiles, r = tile - g * group_tiles;
    const uint32_t width = min(group_n, tiles_n - g * group_n);
    mi = r / width;
    ni = g * group_n + (r - mi * width);
}

// Tensor maps of the three bf16 parts of both operands (SPLIT kernels only).
//
// SPLIT kernels keep the running sum in registers, not in TMEM: the tensor pipe truncates (does not round)
// when it adds into an f32 accumulator, one truncation per instruction, and over a long K that bias reaches
// 1e-5 .. 1e-4 of the result. So the MMA warp closes its accumulators after every kSplitFlush K steps and the
// epilogue warps add them to 64 registers per thread with round-to-nearest f32 adds. A close has TWO
// accumulators of 128 columns: the five small pairs go to one (its sum is 2^-8 of the result, so its
// truncations do not count), the leading pair (part 0 x part 0) to the other, which therefore takes only
// 4 * kSplitFlush = 32 instructions per close: the truncation bias is -7e-7 of the result whatever K is
// (-3e-7 with 4 K steps per close, which left the MMA warp waiting behind the heavier epilogues). Two closes
// fit TMEM, so the MMA warp runs up to 2 * kSplitFlush K steps ahead of the epilogue warps (about as long as
// a tile's epilogue, which the same warps run). The tile is 128 x 128.
// One pipeline stage of a SPLIT kernel holds one K step of ALL six part tiles (3 of A, 3 of B, 16 KiB each), so
// every part is fetched once per K step and used by up to three of the six products; fetching per product
// (twelve tiles per K step) left the tensor pipe 45 % busy, waiting for L2.
struct TcSplitMaps { CUtensorMap a[3], b[3]; };
constexpr int kSplitPairs = 6;
constexpr uint32_t kSplitFlush = 8;
constexpr uint32_t kSplitPartBytes = kTcBM * kTcBK * 2;          // one part tile: 128 x 64 bf16
constexpr uint32_t kSplitStageBytes = 6 * kSplitPartBytes;      // A0 A1 A2 B0 B1 B2
constexpr uint32_t kSplitStages = 2;
__device__ __forceinline__ int split_a(int p) { return (0x001102 >> (4 * p)) & 0xF; }   // 2,0,1,1,0,0
__device__ __forceinline__ int split_b(int p) { return (0x010120 >> (4 * p)) & 0xF; }   // 0,2,1,0,1,0

template <bool A_MN, bool B_MN, int BN, class Epi, bool SPLIT = false>
__global__ void __launch_bounds__(kTcThreads, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
               uint32_t M, uint32_t N, uint32_t K, uint32_t idesc, uint32_t group_n, Epi epi, TcGate gate,
               int *err_flag, const TcSplitMaps *split_maps) {
    constexpr int NP = SPLIT ? kSplitPairs : 1;   // operand pairs multiplied per K step
    constexpr uint32_t kBufs = 2;                 // accumulator buffers in TMEM (SPLIT: a buffer is a pair, small + leading)
    constexpr uint32_t kBufCols = SPLIT ? 2 * BN : BN;
    static_assert(!SPLIT || BN == 128, "SPLIT kernels use two pairs of 128-column accumulators");
    static_assert(!SPLIT || kSplitStages * kSplitStageBytes <= (uint32_t)(TcShape<BN>::kStages * TcShape<BN>::kStageBytes), "SPLIT stages fit the ring");
    constexpr uint32_t kTmemCols = kBufs * kBufCols;
    using S = TcShape<BN>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t *stages = smem;
    float *epi_buf = reinterpret_cast<float *>(smem + S::kStages * S::kStageBytes);
    uint64_t *full_bar = reinterpret_cast<uint64_t *>(smem + S::kStages * S::kStageBytes + S::kEpiBufBytes);
    uint64_t *empty_bar = full_bar + S::kStages;
    uint64_t *tmem_full = empty_bar + S::kStages;
    uint64_t *tmem_empty = tmem_full + kBufs;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(tmem_empty + kBufs);

    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t tiles_m = (M + kTcBM - 1) / kTcBM, tiles_n = (N + BN - 1) / BN;
    const uint32_t num_tiles = tiles_m * tiles_n;
    const uint32_t num_kb = (K + kTcBK - 1) / kTcBK;

    if (warp == 0 && lane == 0) {
        if (SPLIT) {
            for (int i = 0; i < 3; ++i) { tc::prefetch_tensormap(&split_maps->a[i]); tc::prefetch_tensormap(&split_maps->b[i]); }
        } else {
            tc::prefetch_tensormap(&tmap_a);
            tc::prefetch_tensormap(&tmap_b);
        }
        for (int s = 0; s < S::kStages; ++s) { tc::mbar_init(&full_bar[s], 1); tc::mbar_init(&empty_bar[s], 1); }
        for (uint32_t b = 0; b < kBufs; ++b) { tc::mbar_init(&tmem_full[b], 1); tc::mbar_init(&tmem_empty[b], kTcEpiWarps * 32); }
        tc::fence_barrier_init();
    }
    if (warp == 1) {
        tc::tmem_alloc(tmem_slot, kTmemCols);
        tc::tmem_relinquish();
    }
    tc::tc_fence_before_sync();
    __syncthreads();
    tc::tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ---------------- TMA producer ----------------
        if (lane == 0) {
            uint32_t stage = 0, phase = 0, ready_chunks = 0;
            bool ok = true, gate_ok = true;
            for (uint32_t tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
                uint32_t mi, ni;
                tile_coords(tile, tiles_m, tiles_n, group_n, mi, ni);
                const int32_t m0 = mi * kTcBM, n0 = ni * BN;
                if (gate.flags) {
                    // rows [n0, n0 + BN) of B: the blocks up to the one holding the tile's last row must be in
                    const uint32_t last_row = min((uint32_t)n0 + BN, N) - 1;
                    const uint32_t need = min(gate.chunks, last_row / gate.rows_per_chunk + 1);
                    if (ready_chunks < need) {
                        while (ready_chunks < need && gate_ok) {
                            for (uint32_t r = 0; r < gate.world && gate_ok; ++r)
                                if (r != gate.self) gate_ok = wait_flag_reached(gate.flags + ready_chunks * gate.stride + r, gate.epoch);
                            ++ready_chunks;
                        }
                        if (!gate_ok) { ok = false; break; }
                        tc::fence_proxy_async_all();   // the rows were written through the generic proxy, TMA reads them
                    }
                }
                if constexpr (SPLIT) {
                    for (uint32_t kb = 0; kb < num_kb && ok; ++kb) {
                        if (!tc::mbar_wait(&empty_bar[stage], phase ^ 1)) { ok = false; break; }
                        tc::mbar_arrive_expect_tx(&full_bar[stage], kSplitStageBytes);
                        uint8_t *base = stages + stage * kSplitStageBytes;
                        const int32_t k0 = kb * kTcBK;
#pragma unroll
                        for (int i = 0; i < 3; ++i) {
                            uint8_t *sa = base + i * kSplitPartBytes, *sb = base + (3 + i) * kSplitPartBytes;
                            if (A_MN) {
#pragma unroll
                                for (int j = 0; j < kTcBM / 64; ++j) tc::tma_load_2d(sa + j * 8192, &split_maps->a[i], &full_bar[stage], m0 + j * 64, k0);
                            } else {
                                tc::tma_load_2d(sa, &split_maps->a[i], &full_bar[stage], k0, m0);
                            }
                            if (B_MN) {
#pragma unroll
                                for (int j = 0; j < BN / 64; ++j) tc::tma_load_2d(sb + j * 8192, &split_maps->b[i], &full_bar[stage], n0 + j * 64, k0);
                            } else {
                                tc::tma_load_2d(sb, &split_maps->b[i], &full_bar[stage], k0, n0);
                            }
                        }
                        if (++stage == kSplitStages) { stage = 0; phase ^= 1; }
                    }
                } else {
                    for (uint32_t kb = 0; kb < num_kb && ok; ++kb) {
                        if (!tc::mbar_wait(&empty_bar[stage], phase ^ 1)) { ok = false; break; }
                        tc::mbar_arrive_expect_tx(&full_bar[stage], S::kStageBytes);
                        uint8_t *sa = stages + stage * S::kStageBytes, *sb = sa + kTcABytes;
                        const int32_t k0 = kb * kTcBK;
                        if (A_MN) {
#pragma unroll
                            for (int j = 0; j < kTcBM / 64; ++j) tc::tma_load_2d(sa + j * 8192, &tmap_a, &full_bar[stage], m0 + j * 64, k0);
                        } else {
                            tc::tma_load_2d(sa, &tmap_a, &full_bar[stage], k0, m0);
                        }
                        if (B_MN) {
#pragma unroll
                            for (int j = 0; j < BN / 64; ++j) tc::tma_load_2d(sb + j * 8192, &tmap_b, &full_bar[stage], n0 + j * 64, k0);
                        } else {
                            tc::tma_load_2d(sb, &tmap_b, &full_bar[stage], k0, n0);
                        }
                        if (++stage == S::kStages) { stage = 0; phase ^= 1; }
                    }
                }
            }
            if (!ok) atomicCAS(err_flag, 0, gate_ok ? kTcErrProducer : kTcErrGate);
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            uint32_t stage = 0, phase = 0, acc = 0, acc_phase = 0;
            bool ok = true;
            // An accumulator is closed once per tile, or (SPLIT) every kSplitFlush K steps: see TcSplitMaps.
            const uint32_t closes = SPLIT ? (num_kb + kSplitFlush - 1) / kSplitFlush : 1u;
            for (uint32_t tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
                for (uint32_t cl = 0; cl < closes && ok; ++cl) {
                    if (!tc::mbar_wait(&tmem_empty[acc], acc_phase ^ 1)) { ok = false; break; }
                    tc::tc_fence_after_sync();
                    const uint32_t d_tmem = tmem_base + acc * kBufCols;
                    if constexpr (SPLIT) {
                        const uint32_t d_small = d_tmem, d_lead = d_tmem + BN;
                        const uint32_t steps = min(kSplitFlush, num_kb - cl * kSplitFlush);
                        for (uint32_t st = 0; st < steps; ++st) {
                            if (!tc::mbar_wait(&full_bar[stage], phase)) { ok = false; break; }
                            tc::tc_fence_after_sync();
                            const uint32_t base = tc::smem_u32(stages + stage * kSplitStageBytes);
#pragma unroll
                            for (int p = 0; p < NP; ++p) {   // five small pairs into one accumulator, the leading pair into the other
                                const uint32_t sa = base + split_a(p) * kSplitPartBytes, sb = base + (3 + split_b(p)) * kSplitPartBytes;
                                const bool lead = p == NP - 1;
#pragma unroll
                                for (int j = 0; j < kTcBK / 16; ++j) {
                                    const uint64_t da = A_MN ? tc::make_smem_desc(sa + j * 2048, 8192, 1024)
                                                             : tc::make_smem_desc(sa + j * 32, 16, 1024);
                                    const uint64_t db = B_MN ? tc::make_smem_desc(sb + j * 2048, 8192, 1024)
                                                             : tc::make_smem_desc(sb + j * 32, 16, 1024);
                                    tc::umma_f16(lead ? d_lead : d_small, da, db, idesc, st > 0 || j > 0 || (!lead && p > 0));
                                }
                            }
                            tc::umma_commit(&empty_bar[stage]);
                            if (++stage == kSplitStages) { stage = 0; phase ^= 1; }
                        }
                    } else {
                        for (uint32_t st = 0; st < num_kb; ++st) {
                            if (!tc::mbar_wait(&full_bar[stage], phase)) { ok = false; break; }
                            tc::tc_fence_after_sync();
                            const uint32_t sa = tc::smem_u32(stages + stage * S::kStageBytes), sb = sa + kTcABytes;
#pragma unroll
                            for (int j = 0; j < kTcBK / 16; ++j) {
                                const uint64_t da = A_MN ? tc::make_smem_desc(sa + j * 2048, 8192, 1024)
                                                         : tc::make_smem_desc(sa + j * 32, 16, 1024);
                                const uint64_t db = B_MN ? tc::make_smem_desc(sb + j * 2048, 8192, 1024)
                                                         : tc::make_smem_desc(sb + j * 32, 16, 1024);
                                tc::umma_f16(d_tmem, da, db, idesc, st > 0 || j > 0);
                            }
                            tc::umma_commit(&empty_bar[stage]);      // stage reusable once these MMAs have read it
                            if (++stage == S::kStages) { stage = 0; phase ^= 1; }
                        }
                    }
                    if (!ok) break;
                    tc::umma_commit(&tmem_full[acc]);            // accumulator complete
                    if (++acc == kBufs) { acc = 0; acc_phase ^= 1; }
                }
            }
            if (!ok) atomicCAS(err_flag, 0, kTcErrMma);
        }
    } else {
        // ---------------- epilogue ----------------
        const uint32_t ew = warp - 2;                 // 0..7
        const uint32_t quarter = warp & 3;            // TMEM lanes this warp may read: 32*quarter ..
        const uint32_t half = ew >> 2;                // which half of the tile's columns
        float *buf = epi_buf + ew * (32 * 33);
        uint32_t acc = 0, acc_phase = 0;
        bool ok = true;
        for (uint32_t tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
            uint32_t mi, ni;
            tile_coords(tile, tiles_m, tiles_n, group_n, mi, ni);
            const uint32_t m0 = mi * kTcBM, n0 = ni * BN;
            float part[2][32];                        // SPLIT: this thread's row, its 64 columns, summed over K
            if constexpr (SPLIT) {
#pragma unroll
                for (int j = 0; j < 32; ++j) part[0][j] = part[1][j] = 0.0f;
                for (uint32_t cl = 0; cl < (num_kb + kSplitFlush - 1) / kSplitFlush && ok; ++cl) {
                    if (!tc::mbar_wait(&tmem_full[acc], acc_phase)) { ok = false; break; }
                    tc::tc_fence_after_sync();
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
#pragma unroll
                        for (int which = 0; which < 2; ++which) {   // the leading pair's sum, then the small pairs'
                            float t[32];
                            tc::tmem_ld_32x32(tmem_base + ((quarter * 32) << 16) + acc * kBufCols + (1 - which) * BN + half * (BN / 2) + h * 32, t);
#pragma unroll
                            for (int j = 0; j < 32; ++j) part[h][j] += t[j];
                        }
                    }
                    tc::tc_fence_before_sync();
                    tc::mbar_arrive(&tmem_empty[acc]);
                    if (++acc == kBufs) { acc = 0; acc_phase ^= 1; }
                }
                if (!ok) break;
            } else {
                if (!tc::mbar_wait(&tmem_full[acc], acc_phase)) { ok = false; break; }
                tc::tc_fence_after_sync();
            }
            // Runs of a 32-column chunk: pass p covers rows 8p + lane/4, columns 8*(lane%4) .. +8. The
            // fast path (128-bit accesses, a full run of 8 columns) keeps the global loads of the NEXT
            // group of G passes in flight while the current group is finished, also across chunks, so
            // that only the first group of a tile waits for memory with nothing else to do.
            // Generic functors (every activation and normalisation case in one body) run the group loop
            // rolled, because their body must exist once or the kernel outgrows the instruction cache;
            // the price is that handing `nxt` over to `cur` at the end of an iteration waits for the
            // loads. Specialised functors are small enough to unroll the loop (4 bodies): two register
            // sets then swap roles and nothing waits before the data is needed.
            constexpr int G = EpiGroup<Epi>::value, NQ = 4 / G;
            constexpr bool kPing = EpiPingPong<Epi>::value;
            static_assert(!kPing || NQ % 2 == 0, "ping-pong needs an even number of groups per chunk");
            const uint32_t c_end = (half + 1) * (BN / 2);
            const uint32_t cc = (lane & 3) * 8;
            const uint32_t row_base = m0 + quarter * 32 + (lane >> 2);
            typename Epi::Cols cols, cols_n;
            typename Epi::Pre pre[2][G];              // [0]: current group at the start of a chunk
            bool have = false;                        // pre[0] / cols already hold this chunk's first group
#pragma unroll 1
            for (uint32_t c0 = half * (BN / 2); c0 < c_end; c0 += 32) {
                if (n0 + c0 >= N) break;              // uniform per warp
                const uint32_t col = n0 + c0 + cc;
                const bool col_ok = col < N;
                const uint32_t ncols = col_ok ? min(8u, N - col) : 0u;
                const bool fast = epi.vec_ok && ncols == 8;   // else: ragged right edge, unaligned tensors
                if (fast && !have) {
                    epi.cols(col, cols);
#pragma unroll
                    for (int g = 0; g < G; ++g)
                        if (row_base + 8 * g < M) epi.prefetch(row_base + 8 * g, col, pre[0][g]);
                }
                float v[32];
                if constexpr (SPLIT) {
                    const bool first = c0 == half * (BN / 2);
#pragma unroll
                    for (int j = 0; j < 32; ++j) v[j] = first ? part[0][j] : part[1][j];
                } else {
                    tc::tmem_ld_32x32(tmem_base + ((quarter * 32) << 16) + acc * kBufCols + c0, v);
                }
#pragma unroll
                for (int j = 0; j < 32; ++j) buf[lane * 33 + j] = v[j];
                __syncwarp();
                bool have_n = false;
                typename EpiAcc<Epi>::type sums;
                if constexpr (EpiAcc<Epi>::value) epi.acc_init(sums);
                auto group = [&](int q, typename Epi::Pre (&cur)[G], typename Epi::Pre (&nxt)[G]) {
                    if (fast) {
                        if (q + 1 < NQ) {
#pragma unroll
                            for (int g = 0; g < G; ++g) {
                                const uint32_t row = row_base + 8 * ((q + 1) * G + g);
                                if (row < M) epi.prefetch(row, col, nxt[g]);
                            }
                        } else if (c0 + 32 < c_end && col + 40 <= N) {   // first group of the next chunk
                            epi.cols(col + 32, cols_n);
#pragma unroll
                            for (int g = 0; g < G; ++g)
                                if (row_base + 8 * g < M) epi.prefetch(row_base + 8 * g, col + 32, nxt[g]);
                            have_n = true;
                        }
                    }
#pragma unroll
                    for (int g = 0; g < G; ++g) {
                        const uint32_t rr = (q * G + g) * 8 + (lane >> 2), row = m0 + quarter * 32 + rr;
                        float r[8];
#pragma unroll
                        for (int j = 0; j < 8; ++j) r[j] = buf[rr * 33 + cc + j];
                        if (col_ok && row < M) {
                            if (fast) {
                                if constexpr (EpiAcc<Epi>::value) epi.finish(row, col, r, cur[g], cols, sums);
                                else epi.finish(row, col, r, cur[g], cols);
                            } else {
                                epi.template run<8>(row, col, r, ncols);
                            }
                        }
                    }
                };
                if constexpr (kPing) {
#pragma unroll
                    for (int q = 0; q < NQ; ++q) group(q, pre[q & 1], pre[(q + 1) & 1]);
                } else {
#pragma unroll 1
                    for (int q = 0; q < NQ; ++q) {
                        group(q, pre[0], pre[1]);
#pragma unroll
                        for (int g = 0; g < G; ++g) pre[0][g] = pre[1][g];
                    }
                }
                if constexpr (EpiAcc<Epi>::value) epi.acc_flush(sums, (m0 + quarter * 32) / 32, col, lane, fast);
                if (have_n) cols = cols_n;
                have = have_n;
                __syncwarp();
            }
            if constexpr (!SPLIT) {
                tc::tc_fence_before_sync();
                tc::mbar_arrive(&tmem_empty[acc]);
                if (++acc == kBufs) { acc = 0; acc_phase ^= 1; }
            }
        }
        if (!ok && lane == 0) atomicCAS(err_flag, 0, kTcErrEpilogue);
    }

    tc::tc_fence_before_sync();
    __syncthreads();
    tc::tc_fence_after_sync();
    if (warp == 1) tc::tmem_dealloc(tmem_base, kTmemCols);
}

} // namespace sk
