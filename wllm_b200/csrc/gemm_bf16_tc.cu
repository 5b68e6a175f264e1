// bfloat16 matrix product on the fifth-generation tensor cores:
//     C[M, N] = A[M, K] * W[N, K]^T        (both operands K-major, 32-bit accumulation in TMEM)
//
// One persistent CTA per SM walks 128 x 256 output tiles.  Roles by warp:
//   warp 0      one lane issues TMA loads (cp.async.bulk.tensor, 128-byte swizzle) of a 128 x 64 tile
//               of A and two 128 x 64 tiles of W per stage into a ring of four to six stages in shared
//               memory;
//   warp 1      allocates the 512 columns of tensor memory (two 128 x 256 fp32 accumulators); one lane
//               issues tcgen05.mma (M 128, N 256, K 16) on shared-memory descriptors and frees each
//               stage with tcgen05.commit;
//   warps 2-5   read a finished accumulator with tcgen05.ld (each warp its own 32 lanes), apply the
//               epilogue and store, while the next tile's products fill the other accumulator.
// Epilogues: bfloat16 C; 32-bit C (logits); or the gated feed-forward activation, for which the two
// W tiles of a stage are rows n..n+127 of the gate matrix and of the up matrix (W = [gate; up]), so
// that act(gate) * up leaves the kernel and the [M, 2I] intermediate is never written.
//
// Every wait on an mbarrier is bounded: after WAIT_LIMIT failed polls the waiting role records a code
// in `status`, stops, and the CTA leaves through the common exit, where tensor memory is freed.
// Rows of A or W outside the matrices are zero-filled by the TMA unit, so any M and N are taken; K and
// the row pitches must be multiples of 8 elements (16-byte TMA strides).
#include "tc_common.cuh"

#include <mutex>
#include <unordered_map>

constexpr int BM = 128, BN = 256, BK = 64, UMMA_K = 16;
constexpr int B_HALF_BYTES = 128 * BK * 2, B_BYTES = 2 * B_HALF_BYTES;
// A product of few rows loads only AROWS (32, 64 or 128) rows of A per stage; the tensor core still reads
// 128 rows from that address, and the rows past AROWS (whatever lies behind in shared memory) only reach
// accumulator rows that are never stored.  The smaller stage buys a deeper ring: more weight bytes in
// flight per SM, which is what a step bound by streaming the weights needs.
// The W tile of a stage is two halves of `half_rows` rows (a multiple of 16, at most 128): rows n.. and
// n + half_rows.. of W, or the same rows of the gate and of the up matrix.  The host picks half_rows so that
// the tiles (times the parts of K) fill the SMs evenly; smaller halves make the stages smaller and the ring
// deeper (the stage count is fixed at launch from the ring's bytes).
template <int AROWS> struct Ring {
    static constexpr int A_BYTES = AROWS * BK * 2;
    static constexpr int RING_BYTES = (AROWS == 128 ? 4 : (AROWS == 64 ? 5 : 6)) * (A_BYTES + B_BYTES);
    static constexpr int MAX_STAGES = 12;
    static constexpr int SMEM_BYTES = RING_BYTES + 1024 /* alignment slack */ + 256 /* barriers */;
};
constexpr int NUM_THREADS = 192;

enum { EPI_BF16 = 0, EPI_F32 = 1, EPI_GATED_GELU = 2, EPI_GATED_SILU = 3 };
// With k_splits > 1 (32-bit output only) the K range is cut into k_splits parts of whole 64-column
// blocks; part s of a tile is a work item of its own and writes its partial sum to slab s of C
// ([k_splits][M][ldc]).  Whoever reads C adds the slabs in order (the norm and rotary kernels do), so the
// result does not depend on which CTA ran which part.  This is how a step of a few rows keeps every SM
// streaming weights.  (Letting the CTA that finishes a tile last add the slabs inside this kernel was
// tried and measured slower: the sum then runs on one SM at the tail of the kernel.)

// status codes written by a role that gave up waiting
enum { GAVE_UP_PRODUCER = 11, GAVE_UP_MMA = 12, GAVE_UP_EPILOGUE = 13 };


// gelu_tanh(x) = x/2 (1 + tanh u) = x / (1 + e^(-2u)),  u = sqrt(2/pi) (x + 0.044715 x^3): one exponential
// and one division instead of a tanh.
__device__ __forceinline__ float epi_gelu(float x) {
    const float u = 0.7978845608028654f * (x + 0.044715f * x * x * x);
    return __fdividef(x, 1.0f + __expf(-2.0f * u));
}
__device__ __forceinline__ float epi_silu(float x) { return __fdividef(x, 1.0f + __expf(-x)); }

// Epilogue of one warp for one tile: reads its 32 lanes of the accumulator at t_acc (tile_n columns, a
// multiple of 16; for the gated epilogues gate in columns 0.. and up from column up_col), applies the
// epilogue and stores rows m0 + 32 * quarter + lane of C.
template <int EPI, int W>
__device__ __forceinline__ void drain_chunk(void* __restrict__ c, int ldc, int M, int n_cols, int split, int row, int col,
                                            uint32_t t_chunk, uint32_t up_col) {
    constexpr bool GATED = EPI == EPI_GATED_GELU || EPI == EPI_GATED_SILU;
    uint32_t v[W];
    float f[W];
    tc_ld<W>(t_chunk, v);
    if (GATED) {
        uint32_t u[W];
        tc_ld<W>(t_chunk + up_col, u);
        tc_wait_ld();
#pragma unroll
        for (int i = 0; i < W; ++i) {
            const float g = __uint_as_float(v[i]);
            f[i] = (EPI == EPI_GATED_GELU ? epi_gelu(g) : epi_silu(g)) * __uint_as_float(u[i]);
        }
    } else {
        tc_wait_ld();
#pragma unroll
        for (int i = 0; i < W; ++i) f[i] = __uint_as_float(v[i]);
    }
    if (row >= M) return;
    if (EPI == EPI_F32) {
        float* dst = reinterpret_cast<float*>(c) + ((size_t)split * M + row) * ldc + col;
        if (col + W <= n_cols && (ldc & 3) == 0) {
#pragma unroll
            for (int i = 0; i < W; i += 4)
                *reinterpret_cast<float4*>(dst + i) = make_float4(f[i], f[i + 1], f[i + 2], f[i + 3]);
        } else {
            for (int i = 0; i < W; ++i)
                if (col + i < n_cols) dst[i] = f[i];
        }
    } else {
        bf16* dst = reinterpret_cast<bf16*>(c) + (size_t)row * ldc + col;
        if (col + W <= n_cols && (ldc & 7) == 0) {
#pragma unroll
            for (int i = 0; i < W; i += 8) {
                uint4 o;
                __nv_bfloat162 p0 = __floats2bfloat162_rn(f[i], f[i + 1]), p1 = __floats2bfloat162_rn(f[i + 2], f[i + 3]);
                __nv_bfloat162 p2 = __floats2bfloat162_rn(f[i + 4], f[i + 5]), p3 = __floats2bfloat162_rn(f[i + 6], f[i + 7]);
                o.x = *reinterpret_cast<uint32_t*>(&p0); o.y = *reinterpret_cast<uint32_t*>(&p1);
                o.z = *reinterpret_cast<uint32_t*>(&p2); o.w = *reinterpret_cast<uint32_t*>(&p3);
                *reinterpret_cast<uint4*>(dst + i) = o;
            }
        } else {
            for (int i = 0; i < W; ++i)
                if (col + i < n_cols) dst[i] = __float2bfloat16_rn(f[i]);
        }
    }
}

template <int EPI>
__device__ __forceinline__ void drain_accumulator(void* __restrict__ c, int ldc, int M, int n_cols, int tile_n, int up_col,
                                                  int split, int m0, int n0, uint32_t t_acc, int quarter, int lane) {
    const int row = m0 + quarter * 32 + lane;
    const uint32_t t_row = t_acc + ((uint32_t)(quarter * 32) << 16);
    if (m0 + quarter * 32 >= M) return;                      // the same for the whole warp
    int c0 = 0;
#pragma unroll 1
    for (; c0 + 32 <= tile_n; c0 += 32) drain_chunk<EPI, 32>(c, ldc, M, n_cols, split, row, n0 + c0, t_row + c0, up_col);
    if (c0 < tile_n) drain_chunk<EPI, 16>(c, ldc, M, n_cols, split, row, n0 + c0, t_row + c0, up_col);
}

template <int EPI, int AROWS>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w, void* __restrict__ c,
               int ldc, int M, int N, int K, int up_row_offset, int k_splits, int half_rows, int* __restrict__ status) {
    constexpr int A_BYTES = Ring<AROWS>::A_BYTES, RING_BYTES = Ring<AROWS>::RING_BYTES, MAX_STAGES = Ring<AROWS>::MAX_STAGES;
    const int B_HALF = half_rows * BK * 2, STAGE_BYTES = A_BYTES + 2 * B_HALF;
    const int STAGES = min(MAX_STAGES, RING_BYTES / STAGE_BYTES);
    extern __shared__ unsigned char smem_raw[];
    // ring at a 1024-byte boundary (swizzle atoms), barriers behind it
    const uint32_t ring = (smem_addr(smem_raw) + 1023u) & ~1023u;
    const uint32_t bars = ring + RING_BYTES;
    const uint32_t full0 = bars, empty0 = bars + 8 * MAX_STAGES, tfull0 = bars + 16 * MAX_STAGES, tempty0 = tfull0 + 16;
    const uint32_t tmem_slot = tempty0 + 16;
    volatile uint32_t* tmem_slot_ptr = reinterpret_cast<volatile uint32_t*>(smem_raw + (tmem_slot - smem_addr(smem_raw)));

    pdl_launch_dependents();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    constexpr bool GATED = EPI == EPI_GATED_GELU || EPI == EPI_GATED_SILU;
    const int n_cols = GATED ? N / 2 : N;                       // columns of the output
    const int tile_n = GATED ? half_rows : 2 * half_rows;       // output columns per tile
    const int UP_COL = half_rows;                               // accumulator column where the second half begins
    const uint32_t idesc = umma_idesc(BM, 2 * half_rows, false, false);
    const int tiles_m = (M + BM - 1) / BM, tiles_n = (n_cols + tile_n - 1) / tile_n;
    const int tiles_mn = tiles_m * tiles_n, num_tiles = tiles_mn * k_splits;
    const int kblocks = (K + BK - 1) / BK, kb_per = (kblocks + k_splits - 1) / k_splits;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(full0 + 8 * s, 1); mbar_init(empty0 + 8 * s, 1); }
        for (int a = 0; a < 2; ++a) { mbar_init(tfull0 + 8 * a, 1); mbar_init(tempty0 + 8 * a, 4); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tmem_slot), "r"(512) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot_ptr;

    if (warp == 0) {
        // ---------------- TMA producer ----------------
        if (lane == 0) {
            uint32_t stage = 0, phase = 0;
            bool ok = true;
            // With one tile of rows every weight is read once in this launch: its lines go first when the L2
            // needs room.  With more tiles of rows the L2 serves the weights to the later ones.
            const bool once = tiles_m == 1;
            const uint64_t stream = l2_evict_first();
            auto load_w = [&](uint32_t dst, uint32_t bar, int x, int y) {
                if (once) tma_load_2d_hint(dst, &map_w, bar, x, y, stream);
                else tma_load_2d(dst, &map_w, bar, x, y);
            };
            // The weights are written by no kernel of the step: the first stages' W tiles are requested before
            // this kernel waits for its predecessor, so they stream while that kernel still runs.  A (the
            // activations the predecessor wrote) follows after the wait.
            int early = 0;
            if (blockIdx.x < num_tiles) {
                const int tile = blockIdx.x;
                const int mn = tile % tiles_mn, split = tile / tiles_mn;
                const int n0 = (mn / tiles_m) * tile_n;
                const int kb_lo = split * kb_per, kb_hi = min(kblocks, kb_lo + kb_per);
                early = min(STAGES, kb_hi - kb_lo);
                for (int i = 0; i < early; ++i) {
                    const uint32_t b_dst = ring + i * STAGE_BYTES + A_BYTES, bar = full0 + 8 * i;
                    mbar_expect_tx(bar, STAGE_BYTES);
                    load_w(b_dst, bar, (kb_lo + i) * BK, n0);
                    load_w(b_dst + B_HALF, bar, (kb_lo + i) * BK, GATED ? up_row_offset + n0 : n0 + half_rows);
                }
            }
            pdl_wait();
            int issued = 0;
            for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
                const int mn = tile % tiles_mn, split = tile / tiles_mn;
                const int m0 = (mn % tiles_m) * BM, n0 = (mn / tiles_m) * tile_n;
                const int kb_lo = split * kb_per, kb_hi = min(kblocks, kb_lo + kb_per);
                for (int kb = kb_lo; kb < kb_hi; ++kb, ++issued) {
                    const uint32_t a_dst = ring + stage * STAGE_BYTES, b_dst = a_dst + A_BYTES, bar = full0 + 8 * stage;
                    if (issued < early) {
                        tma_load_2d(a_dst, &map_a, bar, kb * BK, m0);       // W of this stage is already on its way
                    } else {
                        if (!mbar_wait(empty0 + 8 * stage, phase ^ 1)) { ok = false; break; }
                        mbar_expect_tx(bar, STAGE_BYTES);
                        tma_load_2d(a_dst, &map_a, bar, kb * BK, m0);
                        load_w(b_dst, bar, kb * BK, n0);
                        load_w(b_dst + B_HALF, bar, kb * BK, GATED ? up_row_offset + n0 : n0 + half_rows);
                    }
                    if (++stage == STAGES) { stage = 0; phase ^= 1; }
                }
            }
            if (!ok) atomicExch(status, GAVE_UP_PRODUCER);
            // Loads still in flight land in this CTA's shared memory: stay until every stage that was
            // filled has been consumed (its `empty` phase completes), or the limit passes.
            for (int s = 0; s < STAGES; ++s) {
                if (!mbar_wait(empty0 + 8 * stage, phase ^ 1)) break;
                if (++stage == STAGES) { stage = 0; phase ^= 1; }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            uint32_t stage = 0, phase = 0, it = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++it) {
                const uint32_t acc = it & 1, acc_phase = (it >> 1) & 1;
                if (!mbar_wait(tempty0 + 8 * acc, acc_phase ^ 1)) { ok = false; break; }
                tc_fence_after();
                const uint32_t d = tmem_base + acc * BN;
                const int split = tile / tiles_mn;
                const int kb_lo = split * kb_per, kb_hi = min(kblocks, kb_lo + kb_per);
                for (int kb = kb_lo; kb < kb_hi; ++kb) {
                    if (!mbar_wait(full0 + 8 * stage, phase)) { ok = false; break; }
                    tc_fence_after();
                    const uint32_t a_src = ring + stage * STAGE_BYTES, b_src = a_src + A_BYTES;
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k)
                        tc_mma(d, smem_desc(a_src + k * UMMA_K * 2), smem_desc(b_src + k * UMMA_K * 2), idesc,
                               (kb > kb_lo || k > 0) ? 1u : 0u);
                    tc_commit(empty0 + 8 * stage);          // the stage is free once these products are done
                    if (++stage == STAGES) { stage = 0; phase ^= 1; }
                }
                if (ok) tc_commit(tfull0 + 8 * acc);        // the accumulator is complete
            }
            if (!ok) atomicExch(status, GAVE_UP_MMA);
        }
    } else {
        // ---------------- epilogue: warps 2..5, each its own quarter of the 128 lanes ----------------
        pdl_wait();                  // C may still be read by the kernel before this one
        const int quarter = warp & 3;
        uint32_t it = 0;
        bool ok = true;
        for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++it) {
            const uint32_t acc = it & 1, acc_phase = (it >> 1) & 1;
            const int mn = tile % tiles_mn, split = tile / tiles_mn;
            const int m0 = (mn % tiles_m) * BM, n0 = (mn / tiles_m) * tile_n;
            if (!mbar_wait(tfull0 + 8 * acc, acc_phase)) { ok = false; break; }
            tc_fence_after();
            drain_accumulator<EPI>(c, ldc, M, n_cols, tile_n, UP_COL, split, m0, n0, tmem_base + acc * BN, quarter, lane);
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(tempty0 + 8 * acc);   // this warp has drained its quarter
        }
        if (!ok && lane == 0) atomicExch(status, GAVE_UP_EPILOGUE);
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512) : "memory");
    }
}

// ------------------------------------------------------------------------------------------------
// Two CTAs per tile.  A cluster of two CTAs (on neighbouring SMs) shares a 256 x 256 tile: each holds its
// own 128 rows of A and ONE half of the W tile (128 of the 256 rows), and tcgen05.mma.cta_group::2, issued
// by the first CTA for both, multiplies each CTA's A rows by both halves.  A stage is then 32 KB instead
// of 48 KB per CTA, so the ring holds six stages, and each SM writes and reads a third less shared memory
// per product.  Used when A has more than 128 rows.
//   full[s]    lives in the first CTA; both producers announce their bytes there (two arrivals) and both
//              CTAs' copies count on it (cp.async.bulk.tensor with cta_group::2);
//   empty[s]   in each CTA; the issuer's tcgen05.commit arrives on both (commit multicast);
//   tfull[a]   in each CTA, by the same multicast; tempty[a] in the first CTA, eight arrivals (the four
//              epilogue warps of each CTA).
// Both CTAs allocate and free tensor memory together (cta_group::2), and neither leaves before the other
// has finished (cluster barrier): its shared memory and barriers are written by the other until then.
// ------------------------------------------------------------------------------------------------
// Each CTA's half of the W tile has `half_rows` rows (128 unless the host found that another width fills the
// pairs better); narrower halves deepen the ring.  A half of more than 128 rows (up to 256, in steps of 16) makes
// a WIDE tile of 2 * half_rows > 256 output columns: one accumulator instead of two (so the next tile's products
// wait for the drain of this one), two products a step of half_rows columns each, and each CTA's half as two
// boxes of half_rows / 2 rows: rows n0 + rank * half_rows / 2 .. for the first product, the same from
// n0 + half_rows for the second.  It pays where it saves a whole round: 2,048 x 2,560 is 80 tiles of 256 columns
// on 74 pairs, and 72 tiles of 288.
struct PairRing {
    static constexpr int A_BYTES = 128 * BK * 2;
    static constexpr int RING_BYTES = 6 * (A_BYTES + 128 * BK * 2);
    static constexpr int MAX_STAGES = 12;
    static constexpr int SMEM_BYTES = RING_BYTES + 1024 + 256;
};

template <int EPI, bool WIDE>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(NUM_THREADS, 1)
gemm_tc_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w, void* __restrict__ c,
                    int ldc, int M, int N, int K, int up_row_offset, int k_splits, int half_rows, int* __restrict__ status) {
    constexpr int A_BYTES = PairRing::A_BYTES, RING_BYTES = PairRing::RING_BYTES, MAX_STAGES = PairRing::MAX_STAGES;
    const int STAGE_BYTES = A_BYTES + half_rows * BK * 2;
    const int STAGES = min(MAX_STAGES, RING_BYTES / STAGE_BYTES);
    extern __shared__ unsigned char smem_raw[];
    const uint32_t ring = (smem_addr(smem_raw) + 1023u) & ~1023u;
    const uint32_t bars = ring + RING_BYTES;
    const uint32_t full0 = bars, empty0 = bars + 8 * MAX_STAGES, tfull0 = bars + 16 * MAX_STAGES, tempty0 = tfull0 + 16;
    const uint32_t tmem_slot = tempty0 + 16;
    volatile uint32_t* tmem_slot_ptr = reinterpret_cast<volatile uint32_t*>(smem_raw + (tmem_slot - smem_addr(smem_raw)));

    pdl_launch_dependents();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();
    const int pair = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;
    constexpr bool GATED = EPI == EPI_GATED_GELU || EPI == EPI_GATED_SILU;
    const int n_cols = GATED ? N / 2 : N;
    const int tile_n = GATED ? half_rows : 2 * half_rows;
    const int UP_COL = half_rows;
    constexpr bool wide = WIDE;                                // half_rows > 128
    const int part_rows = wide ? half_rows / 2 : half_rows;    // rows of a CTA's half that one product reads
    const uint32_t idesc = umma_idesc(2 * BM, 2 * part_rows, false, false);
    const int tiles_m = (M + 2 * BM - 1) / (2 * BM), tiles_n = (n_cols + tile_n - 1) / tile_n;
    const int tiles_mn = tiles_m * tiles_n, num_tiles = tiles_mn * k_splits;
    const int kblocks = (K + BK - 1) / BK, kb_per = (kblocks + k_splits - 1) / k_splits;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(full0 + 8 * s, 2); mbar_init(empty0 + 8 * s, 1); }
        for (int a = 0; a < 2; ++a) { mbar_init(tfull0 + 8 * a, 1); mbar_init(tempty0 + 8 * a, 8); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) tc_alloc_pair(tmem_slot, 512);
    tc_fence_before();
    cluster_sync();                       // both CTAs' barriers exist before either signals the other
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot_ptr;
    const uint32_t lead_full0 = cluster_map(full0, 0), lead_tempty0 = cluster_map(tempty0, 0);
    // this CTA's half of the W tile: rows n0.. (first CTA) or the second half / the up matrix (second CTA)
    const int w_row_offset = rank == 0 ? 0 : (GATED ? up_row_offset : part_rows);

    if (warp == 0) {
        // ---------------- TMA producer (one in each CTA) ----------------
        if (lane == 0) {
            uint32_t stage = 0, phase = 0;
            bool ok = true;
            int early = 0;
            const bool once = tiles_m == 1;         // one tile of rows: every weight is read once, evicted first
            const uint64_t stream = l2_evict_first();
            auto load_box = [&](uint32_t dst, uint32_t bar, int x, int y) {
                if (once) tma_load_2d_pair_hint(dst, &map_w, bar, x, y, stream);
                else tma_load_2d_pair(dst, &map_w, bar, x, y);
            };
            auto load_w = [&](uint32_t dst, uint32_t bar, int x, int y) {
                load_box(dst, bar, x, y);
                if (wide) load_box(dst + part_rows * BK * 2, bar, x, y + half_rows);
            };
            if (pair < num_tiles) {                 // W tiles of the first stages before the predecessor has finished
                const int mn = pair % tiles_mn, split = pair / tiles_mn;
                const int n0 = (mn / tiles_m) * tile_n;
                const int kb_lo = split * kb_per, kb_hi = min(kblocks, kb_lo + kb_per);
                early = min(STAGES, kb_hi - kb_lo);
                for (int i = 0; i < early; ++i) {
                    mbar_expect_tx_cluster(lead_full0 + 8 * i, STAGE_BYTES);
                    load_w(ring + i * STAGE_BYTES + A_BYTES, lead_full0 + 8 * i, (kb_lo + i) * BK, n0 + w_row_offset);
                }
            }
            pdl_wait();
            int issued = 0;
            for (int tile = pair; tile < num_tiles && ok; tile += num_pairs) {
                const int mn = tile % tiles_mn, split = tile / tiles_mn;
                const int m0 = (mn % tiles_m) * 2 * BM + (int)rank * BM, n0 = (mn / tiles_m) * tile_n;
                const int kb_lo = split * kb_per, kb_hi = min(kblocks, kb_lo + kb_per);
                for (int kb = kb_lo; kb < kb_hi; ++kb, ++issued) {
                    const uint32_t a_dst = ring + stage * STAGE_BYTES, b_dst = a_dst + A_BYTES, bar = lead_full0 + 8 * stage;
                    if (issued < early) {
                        tma_load_2d_pair(a_dst, &map_a, bar, kb * BK, m0);
                    } else {
                        if (!mbar_wait(empty0 + 8 * stage, phase ^ 1)) { ok = false; break; }
                        mbar_expect_tx_cluster(bar, STAGE_BYTES);
                        tma_load_2d_pair(a_dst, &map_a, bar, kb * BK, m0);
                        load_w(b_dst, bar, kb * BK, n0 + w_row_offset);
                    }
                    if (++stage == STAGES) { stage = 0; phase ^= 1; }
                }
            }
            if (!ok) atomicExch(status, GAVE_UP_PRODUCER);
            // stay until every filled stage has been consumed, or the limit passes
            for (int s = 0; s < STAGES; ++s) {
                if (!mbar_wait(empty0 + 8 * stage, phase ^ 1)) break;
                if (++stage == STAGES) { stage = 0; phase ^= 1; }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer: the first CTA's, for both ----------------
        if (lane == 0 && rank == 0) {
            uint32_t stage = 0, phase = 0, it = 0;
            bool ok = true;
            for (int tile = pair; tile < num_tiles && ok; tile += num_pairs, ++it) {
                const uint32_t acc = wide ? 0 : it & 1, acc_phase = (wide ? it : it >> 1) & 1;
                if (!mbar_wait(tempty0 + 8 * acc, acc_phase ^ 1)) { ok = false; break; }
                tc_fence_after();
                const uint32_t d = tmem_base + acc * BN;
                const int split = tile / tiles_mn;
                const int kb_lo = split * kb_per, kb_hi = min(kblocks, kb_lo + kb_per);
                for (int kb = kb_lo; kb < kb_hi; ++kb) {
                    if (!mbar_wait(full0 + 8 * stage, phase)) { ok = false; break; }
                    tc_fence_after();
                    const uint32_t a_src = ring + stage * STAGE_BYTES, b_src = a_src + A_BYTES;
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k) {
                        const uint32_t fresh = (kb > kb_lo || k > 0) ? 1u : 0u;
                        tc_mma_pair(d, smem_desc(a_src + k * UMMA_K * 2), smem_desc(b_src + k * UMMA_K * 2), idesc, fresh);
                        if (wide)
                            tc_mma_pair(d + half_rows, smem_desc(a_src + k * UMMA_K * 2),
                                        smem_desc(b_src + part_rows * BK * 2 + k * UMMA_K * 2), idesc, fresh);
                    }
                    tc_commit_pair(empty0 + 8 * stage, 3);
                    if (++stage == STAGES) { stage = 0; phase ^= 1; }
                }
                if (ok) tc_commit_pair(tfull0 + 8 * acc, 3);
            }
            if (!ok) atomicExch(status, GAVE_UP_MMA);
        }
    } else {
        // ---------------- epilogue: warps 2..5 of each CTA drain that CTA's 128 rows ----------------
        pdl_wait();
        const int quarter = warp & 3;
        uint32_t it = 0;
        bool ok = true;
        for (int tile = pair; tile < num_tiles && ok; tile += num_pairs, ++it) {
            const uint32_t acc = wide ? 0 : it & 1, acc_phase = (wide ? it : it >> 1) & 1;
            const int mn = tile % tiles_mn, split = tile / tiles_mn;
            const int m0 = (mn % tiles_m) * 2 * BM + (int)rank * BM, n0 = (mn / tiles_m) * tile_n;
            if (!mbar_wait(tfull0 + 8 * acc, acc_phase)) { ok = false; break; }
            tc_fence_after();
            drain_accumulator<EPI>(c, ldc, M, n_cols, tile_n, UP_COL, split, m0, n0, tmem_base + acc * BN, quarter, lane);
            tc_fence_before();
            __syncwarp();
            if (lane == 0) {
                if (rank == 0) mbar_arrive(tempty0 + 8 * acc);
                else mbar_arrive_cluster(lead_tempty0 + 8 * acc);
            }
        }
        if (!ok && lane == 0) atomicExch(status, GAVE_UP_EPILOGUE);
    }
    tc_fence_before();
    cluster_sync();                       // nothing of either CTA is still in use by the other
    if (warp == 1) {
        tc_fence_after();
        tc_dealloc_pair(tmem_base, 512);
    }
}

// ------------------------------------------------------------------------------------------------
// host side: tensor maps (cached by what they describe) and the launch
// ------------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiled encoder() {
    static EncodeTiled fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiled>(p);
    }
    return fn;
}

struct MapKey {
    const void* ptr; int rows, cols, ld, box_rows;
    bool operator==(const MapKey& o) const {
        return ptr == o.ptr && rows == o.rows && cols == o.cols && ld == o.ld && box_rows == o.box_rows;
    }
};
struct MapKeyHash {
    size_t operator()(const MapKey& k) const {
        return std::hash<const void*>()(k.ptr) ^ ((size_t)k.rows * 1000003u) ^ ((size_t)k.cols * 10007u) ^
               ((size_t)k.ld << 7) ^ (size_t)k.box_rows;
    }
};
static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> g_maps;
static std::mutex g_maps_mutex;

// Tensor map of a row-major bf16 matrix [rows, cols] with row pitch `ld`, boxes of box_rows rows x 64 columns.
static int tensor_map(const void* ptr, int rows, int cols, int ld, int box_rows, CUtensorMap* out) {
    std::lock_guard<std::mutex> lock(g_maps_mutex);
    const MapKey key{ptr, rows, cols, ld, box_rows};
    auto it = g_maps.find(key);
    if (it != g_maps.end()) { *out = it->second; return WLLM_OK; }
    EncodeTiled enc = encoder();
    if (!enc) return 6;
    const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    const cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
    const cuuint32_t elem[2] = {1, 1};
    CUtensorMap m;
    const CUresult r = enc(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, elem,
                           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return 2000 + (int)r;
    if (g_maps.size() > 4096) g_maps.clear();
    g_maps[key] = m;
    *out = m;
    return WLLM_OK;
}

template <int EPI, int AROWS>
static int launch_rows(const CUtensorMap& ma, const CUtensorMap& mw, void* c, int ldc, int M, int N, int K, int up_off,
                       int k_splits, int half_rows, int* status, int ctas, cudaStream_t stream) {
    // the tensor core reads 128 rows at a stage's A address whatever AROWS is: a stage must hold that many bytes
    if (Ring<AROWS>::A_BYTES + 2 * half_rows * BK * 2 < 128 * BK * 2) return WLLM_BAD_SIZE;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(gemm_tc_kernel<EPI, AROWS>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             Ring<AROWS>::SMEM_BYTES);
        if (e != cudaSuccess) return 1000 + (int)e;
        configured = true;
    }
    return wllm_launch(gemm_tc_kernel<EPI, AROWS>, ctas, NUM_THREADS, Ring<AROWS>::SMEM_BYTES, stream, ma, mw, c, ldc, M, N, K,
                       up_off, k_splits, half_rows, status);
}

// How many pairs can be resident at once.  The kernel is persistent with a fixed stride over the tiles, so
// a pair that only starts when another has left would double the time; not every SM need be part of a
// pair that the hardware can form.
template <int EPI>
static int resident_pairs() {
    static int pairs = -1;
    if (pairs < 0) {
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(2 * 148);
        cfg.blockDim = dim3(NUM_THREADS);
        cfg.dynamicSmemBytes = PairRing::SMEM_BYTES;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        int n = 0;
        // asked of the plain form, whichever form is launched first: it needs its shared memory granted to answer
        cudaFuncSetAttribute(gemm_tc_pair_kernel<EPI, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, PairRing::SMEM_BYTES);
        if (cudaOccupancyMaxActiveClusters(&n, gemm_tc_pair_kernel<EPI, false>, &cfg) != cudaSuccess) { cudaGetLastError(); n = 0; }
        pairs = n;
    }
    return pairs;
}

template <int EPI, bool WIDE>
static int launch_pair_as(const CUtensorMap& ma, const CUtensorMap& mw, void* c, int ldc, int M, int N, int K, int up_off,
                          int k_splits, int half_rows, int* status, int pairs, cudaStream_t stream) {
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(gemm_tc_pair_kernel<EPI, WIDE>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             PairRing::SMEM_BYTES);
        if (e != cudaSuccess) return 1000 + (int)e;
        configured = true;
    }
    const int resident = resident_pairs<EPI>();       // the same for both forms: it is the shared memory that decides
    if (resident < 1) return WLLM_BAD_SIZE;
    if (pairs > resident) pairs = resident;
    return wllm_launch(gemm_tc_pair_kernel<EPI, WIDE>, 2 * pairs, NUM_THREADS, PairRing::SMEM_BYTES, stream, ma, mw, c, ldc, M, N,
                       K, up_off, k_splits, half_rows, status);
}

template <int EPI>
static int launch_pair(const CUtensorMap& ma, const CUtensorMap& mw, void* c, int ldc, int M, int N, int K, int up_off,
                       int k_splits, int half_rows, int* status, int pairs, cudaStream_t stream) {
    constexpr bool GATED = EPI == EPI_GATED_GELU || EPI == EPI_GATED_SILU;
    if constexpr (!GATED) {
        if (half_rows > 128)
            return launch_pair_as<EPI, true>(ma, mw, c, ldc, M, N, K, up_off, k_splits, half_rows, status, pairs, stream);
    }
    return launch_pair_as<EPI, false>(ma, mw, c, ldc, M, N, K, up_off, k_splits, half_rows, status, pairs, stream);
}

// Number of CTA pairs of the two-CTA kernel that one device holds at once (for reports).
WLLM_API int wllm_gemm_bf16_tc_resident_pairs() {
    cudaFuncSetAttribute(gemm_tc_pair_kernel<EPI_BF16, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, PairRing::SMEM_BYTES);
    return resident_pairs<EPI_BF16>();
}

// WLLM_GEMM_PAIR=0 keeps every product on the one-CTA kernel.
static bool pair_enabled() {
    static int on = -1;
    if (on < 0) {
        const char* e = getenv("WLLM_GEMM_PAIR");
        on = (e && e[0] == '0') ? 0 : 1;
    }
    return on != 0;
}

static int a_rows_for(int M) { return M <= 32 ? 32 : (M <= 64 ? 64 : 128); }

template <int EPI>
static int launch(const CUtensorMap& ma, const CUtensorMap& mw, void* c, int ldc, int M, int N, int K, int up_off,
                  int k_splits, int half_rows, int* status, int ctas, cudaStream_t stream) {
    switch (a_rows_for(M)) {
        case 32: return launch_rows<EPI, 32>(ma, mw, c, ldc, M, N, K, up_off, k_splits, half_rows, status, ctas, stream);
        case 64: return launch_rows<EPI, 64>(ma, mw, c, ldc, M, N, K, up_off, k_splits, half_rows, status, ctas, stream);
    }
    return launch_rows<EPI, 128>(ma, mw, c, ldc, M, N, K, up_off, k_splits, half_rows, status, ctas, stream);
}

// C = A W^T.  epilogue 0: bf16 C [M, N]; 1: fp32 C [M, N]; 2 / 3: W = [gate; up] ([N, K], N even), bf16 C [M, N/2]
// = gelu_tanh(gate) * up / silu(gate) * up.  `status` is a device int that stays 0 unless a role gave up waiting.
// k_splits > 1 needs epilogue 1 and a C of k_splits slabs [M, ldc]; every part must hold at least one block of K.
// half_rows (a multiple of 16 up to 128; 0 = 128) sets the width of a tile: 2 * half_rows output columns, or
// half_rows columns of the gated output (by 128 rows, or 256 rows on a pair of CTAs).  On pairs without a gate
// it may also be a multiple of 8, or 144 to 256 in steps of 16 (wide tiles, see the pair kernel).
WLLM_API int wllm_gemm_bf16_tc(const void* a, int lda, const void* w, int ldw, void* c, int ldc, int M, int N, int K,
                               int epilogue, int k_splits, int half_rows, int* status, int max_ctas, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return WLLM_OK;
    if (k_splits < 1 || (k_splits > 1 && epilogue != EPI_F32)) return WLLM_BAD_SIZE;
    {
        const int kblocks = (K + BK - 1) / BK, kb_per = (kblocks + k_splits - 1) / k_splits;
        if (kb_per * (k_splits - 1) >= kblocks && k_splits > 1) return WLLM_BAD_SIZE;   // an empty part
    }
    if (K <= 0 || K % 8 != 0 || lda % 8 != 0 || ldw % 8 != 0 || lda < K || ldw < K) return WLLM_BAD_SIZE;
    if (((uintptr_t)a & 15) || ((uintptr_t)w & 15) || ((uintptr_t)c & 15)) return WLLM_BAD_ALIGN;
    const bool gated = epilogue == EPI_GATED_GELU || epilogue == EPI_GATED_SILU;
    if (gated && (N % 2 != 0)) return WLLM_BAD_SIZE;
    const bool pair = M > BM && max_ctas >= 2 && pair_enabled();
    if (half_rows == 0) half_rows = 128;
    // One-CTA tiles and the gated epilogue drain halves in chunks of 16 columns; a pair's plain tile of two halves
    // takes halves in steps of 8, and wide tiles (two products a step) halves of 144 to 256 in steps of 16.
    const bool wide = half_rows > 128;
    if (wide ? (!pair || gated || half_rows > 256 || half_rows % 16 != 0)
             : (half_rows < 16 || half_rows % ((pair && !gated) ? 8 : 16) != 0))
        return WLLM_BAD_SIZE;
    CUtensorMap ma, mw;
    int r = tensor_map(a, M, K, lda, a_rows_for(M), &ma);
    if (r) return r;
    r = tensor_map(w, N, K, ldw, wide ? half_rows / 2 : half_rows, &mw);
    if (r) return r;
    const int n_cols = gated ? N / 2 : N, tile_n = gated ? half_rows : 2 * half_rows;
    if (pair) {
        const int tiles = ((M + 2 * BM - 1) / (2 * BM)) * ((n_cols + tile_n - 1) / tile_n) * k_splits;
        const int pairs = tiles < max_ctas / 2 ? tiles : max_ctas / 2;
        switch (epilogue) {
            case EPI_BF16: return launch_pair<EPI_BF16>(ma, mw, c, ldc, M, N, K, 0, 1, half_rows, status, pairs, stream);
            case EPI_F32: return launch_pair<EPI_F32>(ma, mw, c, ldc, M, N, K, 0, k_splits, half_rows, status, pairs, stream);
            case EPI_GATED_GELU: return launch_pair<EPI_GATED_GELU>(ma, mw, c, ldc, M, N, K, N / 2, 1, half_rows, status, pairs, stream);
            case EPI_GATED_SILU: return launch_pair<EPI_GATED_SILU>(ma, mw, c, ldc, M, N, K, N / 2, 1, half_rows, status, pairs, stream);
        }
        return WLLM_BAD_SIZE;
    }
    const int tiles = ((M + BM - 1) / BM) * ((n_cols + tile_n - 1) / tile_n) * k_splits;
    const int ctas = tiles < max_ctas ? tiles : max_ctas;
    switch (epilogue) {
        case EPI_BF16: return launch<EPI_BF16>(ma, mw, c, ldc, M, N, K, 0, 1, half_rows, status, ctas, stream);
        case EPI_F32: return launch<EPI_F32>(ma, mw, c, ldc, M, N, K, 0, k_splits, half_rows, status, ctas, stream);
        case EPI_GATED_GELU: return launch<EPI_GATED_GELU>(ma, mw, c, ldc, M, N, K, N / 2, 1, half_rows, status, ctas, stream);
        case EPI_GATED_SILU: return launch<EPI_GATED_SILU>(ma, mw, c, ldc, M, N, K, N / 2, 1, half_rows, status, ctas, stream);
    }
    return WLLM_BAD_SIZE;
}
