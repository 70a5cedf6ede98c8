// Matrix products for prompts on the 5th-generation tensor cores (tcgen05), bfloat16 in, float
// accumulation in tensor memory:   C[m, :] = A[m, :] . B[g(m)]^T
//
//   Two forms of one kernel (template parameter CTAS):
//   * CTAS = 1: a block works on a tile of 128 rows x 256 columns (tcgen05.mma.cta_group::1, M = 128, N = 256);
//   * CTAS = 2: two blocks (a cluster of two CTAs, cta_group::2) work on one tile of 256 rows x 256 columns:
//     each holds its own 128 rows of A and HALF of the B tile (128 of the 256 rows of B) in shared memory, and
//     one tcgen05.mma issued by the leader reads both blocks' operands and writes rows 0..127 of the product
//     into the leader's tensor memory and rows 128..255 into the other's.  Per block and k-block that is 32 KB
//     from L2 for 128 x 256 x 64 of product instead of 48 KB, and six ring stages fit instead of four.
//     Measured when it went in: 1.61 against 1.53 PFLOP/s on 8192 x 4096 x 4096 and +7 % on experts with 2,048 rows
//     each; with few rows per group the 256-row tiles are mostly padding and there are half as many work items
//     (decoding at batch 64: -7 %).  Since the tiles of a group are numbered with its row tiles innermost (tc_tile)
//     the single blocks share their B tiles through L2 just as well, and the launcher takes pairs only from 1,024
//     rows per group on and for a short K (see tb_gemm_tc_bf16);
//   * operands are staged by TMA (cp.async.bulk.tensor, 128-byte swizzle) into a ring of TC_STAGES stages;
//     with pairs, both blocks' copies are counted on the LEADER's barrier of the stage;
//   * tcgen05.commit (with pairs: multicast to both blocks) hands a finished stage back to the TMA warps and, after
//     the last k-block, the accumulator [128 x 256] float (256 TMEM columns, two of them: the next tile's
//     products overlap this tile's epilogue) to both blocks' four epilogue warps, which read it with
//     tcgen05.ld, apply the epilogue in float and store; they hand it back by an arrival on the leader's
//     barrier.  A lane reads one ROW of the accumulator; bfloat16 results therefore pass through a strip of
//     shared memory per warp and leave as whole 128-byte lines (the product with the short K, the experts'
//     down projection, was bound by its row-by-row stores: 68.6 -> 60.4 us at 16 x 512 rows, 0.88 -> 1.15
//     PFLOP/s at 16 x 2,048);
//   Warp roles: 0 = TMA producer, 1 = TMEM allocation (+ MMA issue in the leader), 2..9 = epilogue: a warp reads the
//   32 lanes of tensor memory its number allows (warp % 4), so two warps share each quarter of the rows and take
//   alternate 64-column pieces.  (With four epilogue warps the product with the short K, 11 k-blocks a tile, was bound
//   by its epilogue: the accumulator of a tile took as long to store as the next tile's products to compute.)
//
//   * grouped (the experts, models/llama/common/src/compute.rs:319-330 done as one product per
//     expert over all of its tokens): rows of A are sorted by group; B is the stack of the groups'
//     matrices viewed as one [G * rows, K] tensor; a pair finds its (group, first row) from
//     group_offsets.  Rows of the tile that belong to the next group are computed and not stored.
//   * DUAL (swiglu, compute.rs:324-326): the B tile is 128 gate rows (the leader's half) followed by the
//     128 matching up rows (the other block's), so one N = 256 instruction yields both; the epilogue stores
//     silu(gate) * up.
//   * edges: TMA fills out-of-range rows and the K tail with zeros; stores are predicated.
//
// Every wait on an mbarrier is bounded; a wait that runs out sets *error (nonzero), the block
// stops issuing work, the leader waits (bounded) for the pair's copies in flight, both blocks meet at the
// cluster barrier, free their TMEM and return.
#include <map>
#include <mutex>
#include <tuple>

#include "tc_common.cuh"

#define TC_BM 128                                  // rows of a tile per block; a pair covers 2 * TC_BM
#define TC_BN 256
#define TC_BK 64
#define TC_THREADS 320
#define TC_EPI_WARPS 8                             // two per quarter of the tensor memory's lanes
#define TC_SHARED_GROUPS 256                       // up to this many groups their offsets are kept in shared memory
#define TC_MAX_STAGES 6
#define TC_A_BYTES (TC_BM * TC_BK * 2)
#define TC_BHALF_BYTES (TC_BN / 2 * TC_BK * 2)     // half of the B tile: all that a block of a pair stages
#define TC_STRIP_BYTES (32 * 128)                  // an epilogue warp's strip: 32 rows x 64 bfloat16, on their way out

template <int CTAS> struct TcShape {
    static constexpr int STAGES = CTAS == 2 ? 6 : 4;
    static constexpr int STAGE_BYTES = TC_A_BYTES + (CTAS == 2 ? 1 : 2) * TC_BHALF_BYTES;
    static constexpr int ROWS = CTAS * TC_BM;      // rows of a tile
};

struct TcArgs {
    void* C;
    const int* group_offsets;
    int* error;
    int ldc, M, N, K, G;
    int b_group_rows;   // rows of B per group in the stacked view (N, or 2N when dual)
    int dual;
    int out_float;
    int tiles_m;        // row tiles (with groups: an upper bound; tiles past the last group are skipped)
    int n_tile;         // rows of B in a tile: a multiple of 16 up to TC_BN (fewer when that fills the SMs better)
};

// ---- the kernel ----------------------------------------------------------------------------
// Persistent: a block (or pair) walks the tiles  unit, unit + units, ...  in the order tc_tile gives them (one
// matrix: column tiles of one row tile are neighbours, so concurrent units share its A tile in L2; groups: see
// there).  The TMA ring runs on across tile boundaries.
struct TcTile {
    int g, row0, row_end, n0;
    bool valid;
};

// `offsets`: the groups' row offsets, in shared memory when there are few enough groups (every role of the block
// walks them for every tile: from global memory that is a chain of dependent loads, some 10 us for the last of 16
// groups, on the way to the block's first copy).
__device__ __forceinline__ TcTile tc_tile(const TcArgs& a, const int* offsets, int t, int tiles_n, int n_out, int rows) {
    TcTile r;
    if (!offsets) {
        const int tm = t / tiles_n;
        r.n0 = (t - tm * tiles_n) * n_out;
        r.g = 0;
        r.row0 = tm * rows;
        r.row_end = a.M;
        r.valid = r.row0 < a.M;
        return r;
    }
    // Groups: the tiles of a group are numbered column tile by column tile, the group's row tiles innermost.  Blocks
    // that run at the same time take consecutive numbers, so the few row tiles of a group that need the SAME tile
    // of its weights fetch it together (once from memory, the others from L2), and what they do not share, the
    // group's rows of A, is a few megabytes that stay in L2.  With the row tiles outermost every weight came from
    // memory once per row tile whenever a group's weights exceed L2 (experts 14,336 wide: 235 MB per group,
    // four row tiles: four times the traffic, and the product was bound by it).
    r.valid = false;
    r.g = 0;
    r.row0 = r.row_end = r.n0 = 0;
    int cum = 0;
    for (int g = 0; g < a.G; ++g) {
        const int lo = offsets[g], hi = offsets[g + 1];
        const int tiles_r = (hi - lo + rows - 1) / rows;
        const int n = tiles_r * tiles_n;
        if (t < cum + n) {
            const int local = t - cum;
            const int tn = local / tiles_r, tr = local - tn * tiles_r;
            r.g = g;
            r.row0 = lo + tr * rows;
            r.row_end = hi;
            r.n0 = tn * n_out;
            r.valid = true;
            break;
        }
        cum += n;
    }
    return r;
}

template <int CTAS>
__global__ void __launch_bounds__(TC_THREADS) gemm_tc_kernel(const __grid_constant__ CUtensorMap map_a,
                                                            const __grid_constant__ CUtensorMap map_b,
                                                            const TcArgs a) {
    pdl_sync();
    extern __shared__ uint8_t smem_raw[];
    constexpr int TC_STAGES = TcShape<CTAS>::STAGES, TC_STAGE_BYTES = TcShape<CTAS>::STAGE_BYTES;
    constexpr bool PAIR = CTAS == 2;
    __shared__ __align__(8) uint64_t bars[2 * TC_MAX_STAGES + 4];
    __shared__ uint32_t tmem_slot;
    __shared__ int group_rows[TC_SHARED_GROUPS + 1];
    const int* offsets = a.group_offsets;
    if (a.group_offsets && a.G <= TC_SHARED_GROUPS) {
        for (int i = threadIdx.x; i <= a.G; i += TC_THREADS) group_rows[i] = a.group_offsets[i];
        offsets = group_rows;        // visible to all after the block-wide barrier below
    }
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = PAIR ? cluster_ctarank() : 0;  // 0 leads the pair
    const int pair = blockIdx.x / CTAS, pairs = gridDim.x / CTAS;     // this unit of work and how many there are
    const int n_out = a.dual ? a.n_tile / 2 : a.n_tile; // output columns of a tile
    const int tiles_n = (a.N + n_out - 1) / n_out;
    const uint32_t half_bytes = (uint32_t)(a.n_tile / 2) * TC_BK * 2;      // half of the B tile in shared memory
    const uint32_t stage_tx = TC_A_BYTES + (PAIR ? 1 : 2) * half_bytes;    // bytes one block copies per stage
    const int total = a.tiles_m * tiles_n;
    const int nkb = (a.K + TC_BK - 1) / TC_BK;

    const uint32_t bar0 = smem_u32(bars);
    auto full_bar = [&](int s) { return bar0 + 8u * s; };
    auto empty_bar = [&](int s) { return bar0 + 8u * (TC_MAX_STAGES + s); };
    auto acc_full = [&](int i) { return bar0 + 8u * (2 * TC_MAX_STAGES + i); };
    auto acc_empty = [&](int i) { return bar0 + 8u * (2 * TC_MAX_STAGES + 2 + i); };

    if (threadIdx.x == 0) {
        for (int s = 0; s < TC_STAGES; ++s) {
            mbar_init(full_bar(s), 1);        // the leader's: its producer arms it with both blocks' bytes
            mbar_init(empty_bar(s), 1);       // one multicast commit per use
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(acc_full(i), 1);
            mbar_init(acc_empty(i), TC_EPI_WARPS * CTAS);    // the leader's: one arrival per epilogue warp of every block
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        if (PAIR) tmem_alloc_pair(smem_u32(&tmem_slot), 2 * TC_BN);
        else tmem_alloc(smem_u32(&tmem_slot), 2 * TC_BN);
    }
    tc_fence_before();
    if (PAIR) cluster_sync_all();             // both blocks' barriers exist before either signals the other's
    else __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_slot;

    if (warp == 0) {
        // ---------------- TMA producer (both blocks; bytes are counted on the leader's barrier) ----------------
        if (lane == 0) {
            bool ok = true;
            int it = 0;                       // k-blocks handed to the ring so far, over all tiles
            int s = 0;                        // its stage, and the parity of the stage's last use:
            uint32_t used = 1;                // kept as counters, since this one thread paces the whole block
            for (int t = pair; t < total && ok; t += pairs) {
                const TcTile tl = tc_tile(a, offsets, t, tiles_n, n_out, TcShape<CTAS>::ROWS);
                if (!tl.valid) continue;
                const int a_row = tl.row0 + (int)rank * TC_BM;
                const int b_row = tl.g * a.b_group_rows + tl.n0 + (int)rank * (a.dual ? a.N : a.n_tile / 2);
                for (int kb = 0; kb < nkb && ok; ++kb, ++it) {
                    if (it >= TC_STAGES) ok = mbar_wait(empty_bar(s), used, a.error, 1);
                    if (!ok) break;
                    const uint32_t sa = smem_base + s * TC_STAGE_BYTES, sb = sa + TC_A_BYTES;
                    if (rank == 0) mbar_expect_tx(full_bar(s), CTAS * stage_tx);
                    if (PAIR) {
                        const uint32_t counted = mapa_shared(full_bar(s), 0);
                        tma_load_2d_pair(sa, &map_a, counted, kb * TC_BK, a_row);
                        tma_load_2d_pair(sb, &map_b, counted, kb * TC_BK, b_row);
                    } else {
                        tma_load_2d(sa, &map_a, full_bar(s), kb * TC_BK, a_row);
                        tma_load_2d(sb, &map_b, full_bar(s), kb * TC_BK, b_row);
                        tma_load_2d(sb + half_bytes, &map_b, full_bar(s), kb * TC_BK,
                                    b_row + (a.dual ? a.N : a.n_tile / 2));
                    }
                    if (++s == TC_STAGES) {
                        s = 0;
                        used ^= 1;
                    }
                }
            }
            if (rank == 0 && *(volatile int*)a.error != 0) {
                // something gave up: let the pair's copies land before the blocks go away
                for (int i = max(0, it - TC_STAGES); i < it; ++i)
                    mbar_wait(full_bar(i % TC_STAGES), (i / TC_STAGES) & 1, a.error, 4);
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer: the leader's one thread, for the pair ----------------
        if (lane == 0 && rank == 0) {
            const uint32_t idesc = umma_idesc(TcShape<CTAS>::ROWS, a.n_tile);
            bool ok = true;
            int lt = 0;                       // tiles done by this unit
            int s = 0;                        // the stage of the next k-block and the parity of its use
            uint32_t use = 0;
            for (int t = pair; t < total && ok; t += pairs) {
                const TcTile tl = tc_tile(a, offsets, t, tiles_n, n_out, TcShape<CTAS>::ROWS);
                if (!tl.valid) continue;
                const int buf = lt & 1;
                if (lt >= 2) ok = mbar_wait(acc_empty(buf), ((lt >> 1) - 1) & 1, a.error, 5);   // drained two tiles ago
                if (!ok) break;
                tc_fence_after();
                const uint32_t acc = tmem_base + buf * TC_BN;
                for (int kb = 0; kb < nkb && ok; ++kb) {
                    ok = mbar_wait(full_bar(s), use, a.error, 2);
                    if (!ok) break;
                    tc_fence_after();
                    const uint32_t sa = smem_base + s * TC_STAGE_BYTES, sb = sa + TC_A_BYTES;
                    const uint64_t da = umma_desc(sa), db = umma_desc(sb);
#pragma unroll
                    for (int k = 0; k < TC_BK / 16; ++k)   // 16 bfloat16 = 32 bytes further along K: +2 in units of 16 bytes
                        if (PAIR) umma_bf16_pair(acc, da + 2 * k, db + 2 * k, idesc, (kb | k) != 0);
                        else umma_bf16(acc, da + 2 * k, db + 2 * k, idesc, (kb | k) != 0);
                    // the stage is free (in both blocks) once these MMAs have read it
                    if (PAIR) umma_commit_pair(empty_bar(s), 3);
                    else umma_commit(empty_bar(s));
                    if (++s == TC_STAGES) {
                        s = 0;
                        use ^= 1;
                    }
                }
                // the accumulator is complete (or abandoned), in both blocks
                if (PAIR) umma_commit_pair(acc_full(buf), 3);
                else umma_commit(acc_full(buf));
                ++lt;
            }
        }
    } else {
        // ---------------- epilogue: warps 2..9 of both blocks, TMEM lanes 32 * (warp % 4) ----------------
        const int quad = warp & 3;
        const int piece = (warp - 2) >> 2;      // which of the alternate 64-column pieces this warp takes
        const int row = quad * 32 + lane;
        // bfloat16 results whose rows start on 16-byte boundaries leave through this warp's strip of shared memory
        uint8_t* strip = smem_raw + (smem_base - smem_u32(smem_raw)) + TC_STAGES * TC_STAGE_BYTES + (warp - 2) * TC_STRIP_BYTES;
        const bool wide = !a.out_float && a.N % 8 == 0 && a.ldc % 8 == 0 && (reinterpret_cast<uintptr_t>(a.C) & 15) == 0;
        bool ok = true;
        int lt = 0;
        for (int t = pair; t < total && ok; t += pairs) {
            const TcTile tl = tc_tile(a, offsets, t, tiles_n, n_out, TcShape<CTAS>::ROWS);
            if (!tl.valid) continue;
            const int buf = lt & 1;
            const int m = tl.row0 + (int)rank * TC_BM + row, n0 = tl.n0;
            ok = mbar_wait(acc_full(buf), (lt >> 1) & 1, a.error, 3);
            tc_fence_after();
            if (!ok) break;
            const uint32_t trow = tmem_base + buf * TC_BN + ((uint32_t)(quad * 32) << 16);
            // A warp whose 32 rows all lie beyond the group's rows has nothing to store (with a few rows per group
            // that is most warps of most tiles): it skips the work and only hands the accumulator back.
            const bool any_row = m - lane < tl.row_end;
            for (int c0 = 0; any_row && c0 < n_out; c0 += 32) {
                if (((c0 >> 6) & 1) != piece) continue;
                float v[32];
                tmem_ld32(trow + c0, v);               // warp-collective: every lane takes part
                if (a.dual) {
                    float u[32];
                    tmem_ld32(trow + a.n_tile / 2 + c0, u);
                    // silu(g) * u = g * u / (1 + e^-g) in float, with the hardware's exponential and division
                    // (2 ulp; the result is rounded to bfloat16 next).  The exact forms cost some hundred clocks
                    // per value with only these four warps on the SM to hide them: measured, the epilogue of a tile
                    // took 7 to 18 us, as long as streaming half of the tile's weights.
#pragma unroll
                    for (int i = 0; i < 32; ++i) v[i] = __fdividef(v[i] * u[i], 1.0f + __expf(-v[i]));
                }
                if (wide) {
                    // A lane holds 32 columns of ONE row: stored from here, every instruction of the warp would touch
                    // 32 lines of memory.  So the warp passes two such chunks through its strip of shared memory
                    // (32 rows x 128 bytes; the 16-byte pieces of a row are XOR-swizzled by the row, so that neither
                    // side meets a bank twice) and stores whole 128-byte lines, four rows an instruction.
                    const int half = (c0 >> 5) & 1;
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        __nv_bfloat162 p0 = __floats2bfloat162_rn(v[8 * j], v[8 * j + 1]);
                        __nv_bfloat162 p1 = __floats2bfloat162_rn(v[8 * j + 2], v[8 * j + 3]);
                        __nv_bfloat162 p2 = __floats2bfloat162_rn(v[8 * j + 4], v[8 * j + 5]);
                        __nv_bfloat162 p3 = __floats2bfloat162_rn(v[8 * j + 6], v[8 * j + 7]);
                        uint4 pk;
                        pk.x = *reinterpret_cast<uint32_t*>(&p0);
                        pk.y = *reinterpret_cast<uint32_t*>(&p1);
                        pk.z = *reinterpret_cast<uint32_t*>(&p2);
                        pk.w = *reinterpret_cast<uint32_t*>(&p3);
                        *reinterpret_cast<uint4*>(strip + lane * 128 + (((half * 4 + j) ^ (lane & 7)) << 4)) = pk;
                    }
                    if (half == 1 || c0 + 32 >= n_out) {
                        __syncwarp();
                        const int cb = c0 - half * 32;                       // the strip's first column in the tile
                        const int cols = min(n_out - cb, a.N - n0 - cb);     // its columns that exist (may be <= 0)
                        const int p = lane & 7;
#pragma unroll
                        for (int i = 0; i < 8; ++i) {
                            const int r = (lane >> 3) + 4 * i;
                            const int mr = m - lane + r;
                            if (mr < tl.row_end && 8 * p + 8 <= cols) {       // N is a multiple of 8 here: no torn piece
                                const uint4 pk = *reinterpret_cast<const uint4*>(strip + r * 128 + ((p ^ (r & 7)) << 4));
                                *reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(a.C) + (size_t)mr * a.ldc + n0 + cb +
                                                          8 * p) = pk;
                            }
                        }
                        __syncwarp();
                    }
                    continue;
                }
                const int c_end = min(n_out - c0, a.N - n0 - c0);   // columns of this chunk that exist (may be <= 0)
                if (m < tl.row_end && c_end > 0) {
                    if (a.out_float) {
                        float* dst = static_cast<float*>(a.C) + (size_t)m * a.ldc + n0 + c0;
#pragma unroll
                        for (int i = 0; i < 32; ++i)
                            if (i < c_end) dst[i] = v[i];
                    } else {
                        __nv_bfloat16* dst = static_cast<__nv_bfloat16*>(a.C) + (size_t)m * a.ldc + n0 + c0;
#pragma unroll
                        for (int i = 0; i < 32; ++i)
                            if (i < c_end) dst[i] = __float2bfloat16_rn(v[i]);
                    }
                }
            }
            // this warp has read its lanes of the accumulator: tell the leader's MMA thread
            tc_fence_before();
            __syncwarp();
            if (lane == 0) {
                if (PAIR) mbar_arrive_cluster(mapa_shared(acc_empty(buf), 0));
                else asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(acc_empty(buf)) : "memory");
            }
            ++lt;
        }
    }
    __syncwarp();
    tc_fence_before();
    if (PAIR) cluster_sync_all();             // neither block leaves while the other may still signal it
    else __syncthreads();
    if (warp == 1) {
        if (PAIR) tmem_dealloc_pair(tmem_base, 2 * TC_BN);
        else tmem_dealloc(tmem_base, 2 * TC_BN);
    }
}

// Gather rows: out[m, :] = x[rows[m], :]  (activations sorted by expert, so that TMA can fetch tiles)
__global__ void gather_rows_kernel(const __nv_bfloat16* __restrict__ x, const int* __restrict__ rows,
                                   __nv_bfloat16* __restrict__ out, int d) {
    pdl_sync();
    const int m = blockIdx.x;
    const uint4* src = reinterpret_cast<const uint4*>(x + (size_t)rows[m] * d);
    uint4* dst = reinterpret_cast<uint4*>(out + (size_t)m * d);
    for (int c = threadIdx.x; c < d / 8; c += blockDim.x) dst[c] = src[c];
}

// ---- host side -----------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    });
    return fn;
}

// [rows, K] bfloat16, row pitch ld elements; box = 64 columns x box_rows rows, 128-byte swizzle.
int make_map(CUtensorMap* out, const void* base, long long rows, int K, long long ld, int box_rows) {
    static std::map<std::tuple<const void*, long long, int, long long, int>, CUtensorMap> cache;
    static std::mutex lock;
    std::lock_guard<std::mutex> hold(lock);
    auto key = std::make_tuple(base, rows, K, ld, box_rows);
    auto it = cache.find(key);
    if (it != cache.end()) {
        *out = it->second;
        return 0;
    }
    EncodeTiledFn fn = encode_fn();
    if (!fn) return TB_ERR_UNSUPPORTED;
    cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    cuuint32_t box[2] = {TC_BK, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return TB_ERR_ARG;
    if (cache.size() > 4096) cache.clear();
    cache[key] = *out;
    return 0;
}

static __device__ int tc_error_word;

int* tc_error_ptr() {
    static int* p = nullptr;
    if (!p) {
        const cudaError_t e = cudaGetSymbolAddress((void**)&p, tc_error_word);
        if (e != cudaSuccess) {
            p = nullptr;
            tb_note_error(e);     // the launcher that asked returns this code
        }
    }
    return p;
}

template <int CTAS>
static int tc_launch(const CUtensorMap& ma, const CUtensorMap& mb, TcArgs a, cudaStream_t s) {
    const size_t smem = (size_t)TcShape<CTAS>::STAGES * TcShape<CTAS>::STAGE_BYTES + TC_EPI_WARPS * TC_STRIP_BYTES + 1024;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(gemm_tc_kernel<CTAS>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    const int n_out = a.dual ? a.n_tile / 2 : a.n_tile, rows = TcShape<CTAS>::ROWS;
    a.tiles_m = a.group_offsets ? (a.M + rows - 1) / rows + a.G : (a.M + rows - 1) / rows;
    cudaLaunchConfig_t cfg = {};
    cfg.blockDim = dim3(TC_THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    attr[1].id = cudaLaunchAttributeClusterDimension;
    attr[1].val.clusterDim.x = CTAS;
    attr[1].val.clusterDim.y = 1;
    attr[1].val.clusterDim.z = 1;
    cfg.attrs = attr;
    static int max_units = 0;                  // blocks (or pairs of blocks) that can be resident at once
    if (!max_units) {
        int sms = 0, dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        max_units = sms > 0 ? sms : 1;         // one persistent block per SM
        if (CTAS == 2) {
            int n = 0;
            cfg.gridDim = dim3(sms > 1 ? sms / 2 * 2 : 2);
            cfg.numAttrs = 2;
            const cudaError_t e = cudaOccupancyMaxActiveClusters(&n, gemm_tc_kernel<CTAS>, &cfg);
            if (e != cudaSuccess) {
                cudaGetLastError();
                max_units = 0;                 // asked again at the next launch
                return (int)e;                 // a failed query is an error, not "no room"
            }
            if (n <= 0) {
                max_units = 0;
                return TB_ERR_UNSUPPORTED;     // no room for a pair of these blocks on this device
            }
            max_units = n;
        }
    }
    const int total = a.tiles_m * ((a.N + n_out - 1) / n_out);
    const int units = total < max_units ? total : max_units;
    cfg.gridDim = dim3(CTAS * units);
    cfg.numAttrs = CTAS == 2 ? 2 : 1;
    tb_state_carveout((const void*)gemm_tc_kernel<CTAS>, TC_THREADS, smem);
    cudaLaunchKernelEx(&cfg, gemm_tc_kernel<CTAS>, ma, mb, a);
    return tb_last_error();
}

extern "C" {
// C[m] = A[m] . B[g(m)]^T.  A [M, K] (rows sorted by group), B [G, rows_b, K] with rows_b = N (or 2N when
// out_kind == 2: gate rows then up rows).  out_kind: 0 bfloat16, 1 float, 2 swiglu (bfloat16).
// Refuses (TB_ERR_UNSUPPORTED) what TMA cannot address: K or a pitch that is no multiple of 8,
// a base that is not 16-byte aligned.
int tb_gemm_tc_bf16(const void* A, const void* B, void* C, const int* group_offsets, int lda, int ldb, int ldc, int M,
                    int N, int K, int G, int out_kind, cudaStream_t s) {
    if (M < 0 || N <= 0 || K <= 0 || G <= 0 || out_kind < 0 || out_kind > 2) return TB_ERR_ARG;
    if (K % 8 || lda % 8 || ldb % 8) return TB_ERR_UNSUPPORTED;
    if (((uintptr_t)A | (uintptr_t)B) & 15) return TB_ERR_UNSUPPORTED;
    if (M == 0) return 0;
    const int dual = out_kind == 2;
    const int rows_b = dual ? 2 * N : N;
    // Rows of B per tile: as many column tiles as the full width would need, but of equal widths (N = 688 with
    // swiglu: six tiles of 120 gate and 120 up rows instead of five of 128 and one of 48 padded to 128).
    int n_tile;
    {
        const int out_max = dual ? TC_BN / 2 : TC_BN, unit = dual ? 8 : 16;
        const int tiles = (N + out_max - 1) / out_max;
        const int out = ((N + tiles - 1) / tiles + unit - 1) / unit * unit;
        n_tile = dual ? 2 * out : out;
    }
    // With about one row tile per group (decoding with many sequences: the product streams
    // the experts' weights once and has G x column tiles to spread over the SMs) narrower tiles can fill a round
    // of SMs where the full width leaves a third of them idle; costs in rows loaded per k-block and round.
    if (group_offsets && (long long)M <= (long long)TC_BM * G) {
        static int sms = 0;
        if (!sms) {
            int dev = 0;
            cudaGetDevice(&dev);
            cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
            if (sms <= 0) sms = 1;
        }
        long long best = -1;
        for (int nt = TC_BN; nt >= 64; nt -= 16) {
            const int out = dual ? nt / 2 : nt;
            const long long tiles = (long long)G * ((N + out - 1) / out);
            const long long cost = (tiles + sms - 1) / sms * (64 + nt);
            if (best < 0 || cost < best) {
                best = cost;
                n_tile = nt;
            }
        }
    }
    CUtensorMap ma, mb;
    int rc = make_map(&ma, A, M, K, lda, TC_BM);
    if (rc) return rc;
    rc = make_map(&mb, B, (long long)G * rows_b, K, ldb, n_tile / 2);     // a box is half of the B tile
    if (rc) return rc;
    int* err_ptr = tc_error_ptr();
    if (!err_ptr) return tb_last_error();
    // Pairs of blocks pay from about a thousand rows per group on, and only with a short K (the experts' down
    // product of narrow experts, K = 688: -9 % at 2,048 rows per group), where a tile is over after a few k-blocks
    // and what counts is how few bytes its start needs.  With K = 4,096 both forms measure the same, and with wide
    // experts (K or N of 14,336) the single blocks are 4..20 % faster (1.41 against 1.18 PFLOP/s at 2,048 rows).
    const bool pair = (long long)M >= 1024ll * G && K < 2048;
    TcArgs a{C, group_offsets, err_ptr, ldc, M, N, K, G, rows_b, dual, out_kind == 1, 0, n_tile};
    rc = pair ? tc_launch<2>(ma, mb, a, s) : tc_launch<1>(ma, mb, a, s);
    if (pair && rc == TB_ERR_UNSUPPORTED) rc = tc_launch<1>(ma, mb, a, s);
    return rc;
}

// Nonzero if any tensor-core product gave up on a wait since the last call (1 producer, 2 MMA,
// 3 epilogue, 4 drain, 5 accumulator hand-back); reading it synchronises the device and clears it.
int tb_gemm_tc_status() {
    int v = 0, zero = 0;
    if (cudaMemcpyFromSymbol(&v, tc_error_word, sizeof(int)) != cudaSuccess) return -1;
    if (v) cudaMemcpyToSymbol(tc_error_word, &zero, sizeof(int));
    return v;
}

// The same word copied to `host_dst` (pinned host memory) in stream order, without waiting: it arrives with
// whatever else the caller reads back from that stream, and is not cleared.
int tb_kernel_status_async(int* host_dst, cudaStream_t s) {
    int* p = tc_error_ptr();
    if (!p) return tb_last_error();
    return (int)cudaMemcpyAsync(host_dst, p, sizeof(int), cudaMemcpyDeviceToHost, s);
}

int tb_gather_rows_bf16(const void* x, const int* rows, void* out, int M, int d, cudaStream_t s) {
    if (M < 0 || d <= 0) return TB_ERR_ARG;
    if (d % 8 || (((uintptr_t)x | (uintptr_t)out) & 15)) return TB_ERR_UNSUPPORTED;
    if (M == 0) return 0;
    TB_LAUNCH((gather_rows_kernel), M, 128, 0, s, (const __nv_bfloat16*)x, rows, (__nv_bfloat16*)out, d);
    return tb_last_error();
}
}

// replayable from C++ (tape.h)
#include "tape.h"
TB_TAPE_REGISTER(tb_gemm_tc_bf16)
TB_TAPE_REGISTER(tb_gather_rows_bf16)
