// Tensor-core contraction pass of the parallel mLSTM for sm_100a (tcgen05 MMA, TMEM accumulators,
// TMA-staged 128-byte-swizzled shared-memory tiles).  One kernel template serves the forward and
// the three backward passes (see mlstm_common.cuh for the algebra) and the chunkwise passes (block
// states, forward and backward with a carried state).  It takes the place of the reference's
// mlstm_matmul_kernel (mlstm_matmul.py:37-101), mlstm_matmul_kernel_backward_db (:132-197) and
// mlstm_matmul_kernel_backward (:200-316), of the single-head fp16 kernel mlstm_forward
// (cuda-src/mlstm_forward.cu:12-189) and, in its chunkwise modes, of the scan kernels' contractions
// (mlstm_scan.py:74-137, 200-278).  Head dimensions above 256 are served by scan_gemm.cu.
//
// One CTA owns one stationary 128-row tile (queries in FWD/DQ, keys in DK/DV) of one batch*head
// slice and streams the tiles on the causal side of it.  Warp roles (576 threads):
//   warp 0       TMA producer: stationary tile once per item, then streamed tiles through a ring of slots
//   warp 1       MMA warp and TMEM allocator: the whole warp runs the issue loop, one elected lane issues
//   warps 2-17   four gate groups of four warps: group g turns columns [32g, 32g+32) of every T tile
//                into gated W values, in TMEM (a thread owns one TMEM lane = one row of the tile)
// TMEM (512 columns): T0 [0,128) and T1 [128,256) fp32 128x128; ACC [256, 256+D) fp32.  W overwrites
// T in place: 16-bit W packs two values per column, each group writing over the first 16 of its own
// 32 T columns; 32-bit (tf32) W sits column for column on T.
// The second contraction reads W straight from TMEM as the A operand and the streamed Z tile from
// shared memory as an MN-major B operand, so the gated tile never touches shared or global memory.
//
// What the measurements behind this structure said (in-kernel clock64 stamps, D = 64 ... 256):
//   * tcgen05.mma takes its operands from warp-uniform registers.  Issued from inside an `if (lane == 0)`
//     branch every MMA cost about 100 cycles of issue (a 128x128x16 MMA runs 64); with the warp
//     converged and one elected lane issuing, the tensor pipe itself sets the pace of a batch of MMAs.
//   * Between two batches every instruction of the MMA warp is idle time of the pipe.  Streamed tiles
//     are therefore signalled in whole units (one "loaded" and one "consumed" barrier per unit, the
//     consumed barrier of a Y tile doubling as "T written"), and the barriers of the next batch are
//     tested in the middle of the current one (mbarrier.test_wait; try_wait may suspend the thread).
//   * The gate warps' epilogue (row-sum exchange, accumulator drain, output) sits between two work
//     items with the pipe idle: the exchange and the next item's row terms are moved in front of the
//     accumulator wait, and where shared memory has room the output leaves through TMA stores.
//
// Element types: fp16 / bf16 (kind::f16) and fp32 read as tf32 (kind::tf32).  D is the width this CTA
// contracts over in T and produces in ACC (head dimensions above 256 are served by scan_gemm.cu).
//
// Every wait is bounded: a wait that runs out sets a CTA-wide abort word, every role leaves its
// loop, the CTA stores a non-zero code in the status word, waits a little for copies in flight,
// frees its TMEM and returns.
#include <atomic>
#include <type_traits>

#include "mlstm_common.cuh"
#include "ptx_sm100.cuh"
#include "tc_host.cuh"

namespace mlstm {
namespace {

using namespace ptx;

constexpr int NGROUPS = 4;                      // gate groups: each gates 32 of a T tile's 128 columns
constexpr int NGATE = NGROUPS * 128;            // gate threads
constexpr int NTHREADS = 64 + NGATE;            // + producer warp and MMA warp
constexpr int BOX_BYTES = 128 * 128;  // one TMA box: 128 rows of 128 bytes
constexpr long long WAIT_LIMIT = 4000000000LL;
constexpr float MAX_ROW_EXP2 = 60.0f;           // clamp of the per-row exponent off the diagonal tile (see its use)
constexpr int SLACK_SLEEP_NS = 64;              // poll interval of the roles that wait with slack (gate warps, producer)  // cycles (about two seconds)
// slices whose work items are interleaved in item order: measured at B=16, NH=8, S=4096, D=256 (ms per forward + backward
// step, two runs of three each): 1: 3.70, 2: 3.67, 3: 3.69, 4: 3.60 / 3.62, 6: 3.71, 8: 3.69 / 3.70, 16: 3.74
constexpr int SLICE_SET_DEFAULT = 4;
constexpr int MAX_DEVICES = 64;


template <int D, int ES>
struct TcCfg {
    static constexpr int EPB = 128 / ES;                      // elements per box row
    static constexpr int KSTEP = 32 / ES;                     // contraction elements per MMA
    static constexpr int CHMAX = ES == 2 ? 128 : 64;
    static constexpr int CH = D < CHMAX ? D : CHMAX;          // elements of D per ring slot
    static constexpr int NHALF = D / CH;                      // slots per streamed tile
    static constexpr int SLOT_BYTES = (CH / EPB) * BOX_BYTES;
    static constexpr int X_BYTES = (D / EPB) * BOX_BYTES;
    // Output tiles leave through per-warp staging buffers and TMA stores where shared memory has room for them
    // and a warp's share of a row is 64 bytes or a multiple (16-bit inputs, D = 128); elsewhere from registers.
    static constexpr bool STAGED = (ES == 2 && D == 128);
    static constexpr int STAGE_BYTES = 2048;                  // per gate warp: 32 rows x 64 bytes
    static constexpr int OUT_BYTES = STAGED ? (NGATE / 32) * STAGE_BYTES : 0;
    // (16-bit D = 128: four slots = two steps, which leaves room for the second set of row partials below)
    static constexpr int NSLOT = ES == 2 ? (D == 256 ? 5 : (D == 128 ? 4 : 8)) : (D == 256 ? 3 : (D == 128 ? 5 : 6));
    // Streamed tiles are signalled in units of UH slots: a whole tile where the ring holds at least two tiles,
    // single slots where it does not (tf32 at D = 256: four slots per tile, three in the ring).
    // One "loaded" and one "consumed" barrier per unit, in rings of RING.
    static constexpr int UH = (NSLOT >= 2 * NHALF) ? NHALF : 1;
    static constexpr int UPT = NHALF / UH;                    // units per streamed tile
    static constexpr int RING = 8;                            // >= units in flight (NSLOT / UH)
    static_assert(NSLOT / UH <= RING && NSLOT > UH, "barrier ring too small / unit larger than the slot ring");
    static constexpr int NBAR = 1 + 2 * RING + 2 + 1 + 1 + 1 + 1 + 4;  // x, unit full/consumed, w[2], acc, part, xfree, accfree, item[4]
    // the tiles start at the (1024-byte aligned, checked at run time) base of the dynamic shared memory
    static constexpr int BASE_BYTES = X_BYTES + NSLOT * SLOT_BYTES + OUT_BYTES + NBAR * 8 + 64;
    // row partials [NGROUPS][128], twice (alternating from item to item) where there is room
    static constexpr int PARTS = (BASE_BYTES + 2 * NGROUPS * 128 * 4 <= 232448) ? 2 : 1;
    static constexpr int SMEM_BYTES = BASE_BYTES + PARTS * NGROUPS * 128 * 4;
    static_assert(SMEM_BYTES <= 232448, "exceeds the 227 KB of shared memory a CTA may have");
};


__device__ __forceinline__ uint32_t to_tf32(float x) {
    uint32_t y;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(y) : "f"(x));
    return y;
}

// X3: fp32 operands carried as two bf16 halves each (x = hi + mid to 16 mantissa bits; the split kernel in
// gates.cu writes them side by side as rows of 2 D bf16 values, hi | mid).  Every contraction then issues the
// three products hi*hi + hi*mid + mid*hi into the same fp32 accumulator (kind::f16 MMAs; the dropped mid*mid
// term is 2^-18 relative), and the gated tile W is split the same way in TMEM: a 16-bit W tile fills only
// half of the columns of the T tile it overwrites, the mid halves take the other half.  This gives fp32
// inputs the tensor cores at an accuracy of about 1e-5, where single tf32 products are at 5e-4.
template <int MODE, int D, int ABFMT, typename OutT, bool X3 = false>
// 18 warps = up to 5 per SM sub-partition (16384 registers each): at most 96 registers per thread
__global__ void __launch_bounds__(NTHREADS, 1)
mlstm_tc_pass(const __grid_constant__ CUtensorMap tmX, const __grid_constant__ CUtensorMap tmY,
              const __grid_constant__ CUtensorMap tmZ, const __grid_constant__ CUtensorMap tmI,
              const __grid_constant__ CUtensorMap tmS, const __grid_constant__ CUtensorMap tmO, const PassParams p) {
    constexpr int ES = ABFMT == 2 ? 4 : 2;
    constexpr bool TF32 = ABFMT == 2;
    constexpr int DL = X3 ? 2 * D : D;            // width of the loaded tiles
    using C = TcCfg<DL, ES>;
    using InT = typename std::conditional<ABFMT == 2, float,
                                          typename std::conditional<ABFMT == 1, __nv_bfloat16, __half>::type>::type;
    // element type of the tensors the epilogue reads straight from global memory (output gate, row-dot operand)
    using SideT = typename std::conditional<X3, float, InT>::type;
    static_assert(!X3 || (ABFMT == 1 && (D == 64 || D == 128) && MODE <= DV), "the split form serves D = 64, 128 of the four parallel passes");
    constexpr int BPS = C::CH / 64;               // X3: 128-byte boxes per ring slot
    constexpr int NBX = D / 64;                   // X3: boxes per operand half
    constexpr bool ROWS_ARE_Q = (MODE == FWD || MODE == DQ || MODE == FWDC || MODE == DQC);
    constexpr bool IS_FWD = (MODE == FWD || MODE == FWDC);   // normalised output, row sums kept
    constexpr bool IS_DQ = (MODE == DQ || MODE == DQC);
    constexpr bool IS_DK = (MODE == DK || MODE == DKC);
    // chunkwise passes: the row tile's own block plus one step that applies a carried state
    constexpr bool CHUNKED = (MODE == FWDC || MODE == DQC || MODE == DKC || MODE == DVC);
    static_assert((!CHUNKED && MODE != STATE) || (ES == 2 && (D == 128 || D == 256)),
                  "chunkwise passes are built for 16-bit inputs, D = 128 and 256");
    // A carried state is D x D.  As a streamed operand it comes in D / 128 tiles of 128 key rows, each with its own
    // "state step" (T = the matching 128 columns of the stationary tile through the matching rows of the identity);
    // as the output of STATE it is written in D / 128 work items of 128 key rows each.
    constexpr int NS = CHUNKED ? D / TILE : 0;
    constexpr int NHV = (MODE == STATE) ? D / TILE : 1;

    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t* smem = smem_raw;
    if ((smem_u32(smem) & 1023u) != 0) {  // the swizzled tiles need a 1024-byte aligned base; never seen otherwise
        grid_dep_wait();
        if (threadIdx.x == 0) atomicExch(p.status, 2000);
        return;
    }
    uint8_t* sX = smem;
    uint8_t* sSlot = smem + C::X_BYTES;
    uint8_t* sOut = sSlot + C::NSLOT * C::SLOT_BYTES;   // staging for TMA stores (C::OUT_BYTES, may be empty)
    uint64_t* bars = reinterpret_cast<uint64_t*>(sOut + C::OUT_BYTES);
    uint64_t* bar_x = bars;
    uint64_t* bar_full = bars + 1;              // [RING] unit loaded
    uint64_t* bar_cons = bars + 1 + C::RING;    // [RING] unit consumed: every MMA that reads it has completed.  For the
                                                // last unit of a Y tile this also says "T tile written".
    uint64_t* bar_w = bars + 1 + 2 * C::RING;   // [2] W tile written by the gate groups
    uint64_t* bar_acc = bar_w + 2;              // accumulator complete
    uint64_t* bar_part = bar_acc + 1;           // row partials of both gate groups in shared memory
    uint64_t* bar_xfree = bar_part + 1;         // stationary tile no longer read by the item's contractions
    uint64_t* bar_accfree = bar_xfree + 1;      // accumulator drained by the item's epilogue
    uint64_t* bar_item = bar_accfree + 1;       // [4] work item published by the producer
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + C::NBAR);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    volatile int* item_ids = reinterpret_cast<volatile int*>(tmem_slot + 2);  // [4] ring of published work items
    // [PARTS][NGROUPS][128]: row sums in FWD / STATE, row dots in DQ / DK, one value per gate group and row
    float* part_base = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(bars) + C::NBAR * 8 + 64);
    constexpr bool STAGED = C::STAGED && !X3;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int NT = p.Spad / TILE;
    const int per_slice = (MODE == STATE) ? p.NB * NHV : NT;     // work items per batch*head slice
    const int total = per_slice * p.BH;

    // A work item = one stationary tile (STATE: one block) of one slice.  The CTA is persistent and
    // takes the next item from a global counter whenever it is ready for one (the producer thread
    // fetches it and publishes it to the other roles through a four-deep ring in shared memory; it
    // can run at most two items ahead of the slowest role, see the waits on bar_xfree / bar_accfree).
    // Item order: slices in sets of SLICE_SET, inside a set the heaviest tiles first, so that the
    // CTAs running at one time share the K/V (or Q/dH) of a few slices, which stay in L2.
    auto next_item = [&](int n, bool& ok) {   // gate warps (converged)
        ok = mbar_wait_warp<SLACK_SLEEP_NS>(&bar_item[n & 3], (n >> 2) & 1, abort_flag, WAIT_LIMIT);
        return ok ? __shfl_sync(0xffffffffu, item_ids[n & 3], 0) : -1;
    };
    struct Item {
        int bh, tile, blk, first, nsteps, half;
    };
    auto decode = [&](int id) {
        Item it;
        const int x = id;
        const int SLICE_SET = p.slice_set;
        const int per_set = per_slice * SLICE_SET;
        const int set = x / per_set;
        const int within = x - set * per_set;
        const int set_size = min(SLICE_SET, p.BH - set * SLICE_SET);
        const int w = within / set_size;
        it.bh = set * SLICE_SET + (within - w * set_size);
        // tile: the stationary tile (STATE: the block).  nsteps / stream_tile: what is streamed.
        //   FWD, DQ   key tiles 0..tile, diagonal last          DK, DV  query tiles tile..NT-1, diagonal first
        //   FWDC, DQC the first NS steps apply the block's inbound state, then key tiles block_start..tile
        //   DKC, DVC  the first NS steps apply the state carried back from the later blocks, then query tiles tile..block_end
        //   STATE     the block's tiles
        it.tile = (MODE == STATE) ? w / NHV : (ROWS_ARE_Q ? (NT - 1 - w) : w);
        it.half = (MODE == STATE) ? w % NHV : 0;     // STATE: which 128 key rows of the block's state
        it.blk = CHUNKED ? it.tile / p.chunk_tiles : (MODE == STATE ? it.tile : 0);
        it.first = (CHUNKED || MODE == STATE) ? it.blk * p.chunk_tiles : 0;
        const int last = min(it.first + p.chunk_tiles, NT) - 1;   // last tile of the block
        it.nsteps = CHUNKED ? (ROWS_ARE_Q ? (it.tile - it.first + 1 + NS) : (last - it.tile + 1 + NS))
                  : (MODE == STATE) ? (min(p.chunk_tiles, NT - it.first))
                  : (ROWS_ARE_Q ? (it.tile + 1) : (NT - it.tile));
        return it;
    };
    auto stream_tile = [&](const Item& it, int t) {
        if (CHUNKED) return ROWS_ARE_Q ? (it.first + t - NS) : (it.tile + t - NS);  // t >= NS
        if (MODE == STATE) return it.first + t;
        return ROWS_ARE_Q ? t : (it.tile + t);
    };
    auto is_state_step = [&](int t) { return CHUNKED && t < NS; };

    if (threadIdx.x == 0) {
        mbar_init(bar_x, 1);
        mbar_init(bar_xfree, 1);
        for (int s = 0; s < C::RING; s++) {
            mbar_init(&bar_full[s], 1);
            mbar_init(&bar_cons[s], 1);
        }
        mbar_init(&bar_w[0], NGATE / 32);   // one arrival per gate warp
        mbar_init(&bar_w[1], NGATE / 32);
        mbar_init(bar_acc, 1);
        mbar_init(bar_accfree, NGATE / 32);
        mbar_init(bar_part, NGATE / 32);
        for (int k = 0; k < 4; k++) mbar_init(&bar_item[k], 1);
        *abort_flag = 0;
        fence_mbar_init();
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, 512);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t tmem_T0 = tmem_base;
    const uint32_t tmem_ACC = tmem_base + 256;
    // Nothing above touched global memory: with a programmatic launch it ran under the tail of the kernel before this one
    // in the stream.  From here on that kernel's results (gate vectors, counters, earlier passes' outputs) are needed.
    grid_dep_wait();
    grid_dep_launch();

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer
        if (lane == 0) {
            prefetch_tmap(&tmX);
            prefetch_tmap(&tmY);
            prefetch_tmap(&tmZ);
            prefetch_tmap(&tmI);
            prefetch_tmap(&tmS);
            int useq = 0;      // units loaded so far; the MMA warp consumes them in the same order
            bool ok = true;
            // one streamed tile = NHALF slots of CH columns starting at column x0, signalled in units of UH slots
            auto load_tile = [&](const CUtensorMap* map, int x0, int row, int z) {
                for (int un = 0; un < C::UPT && ok; un++, useq++) {
                    uint64_t* fb = &bar_full[useq % C::RING];
                    for (int h2 = 0; h2 < C::UH; h2++) {
                        const int j = useq * C::UH + h2;          // slot sequence number
                        if (j >= C::NSLOT) {                      // the slot's previous unit must have been consumed
                            const int prev = (j - C::NSLOT) / C::UH;
                            ok = mbar_wait<SLACK_SLEEP_NS>(&bar_cons[prev % C::RING], (prev / C::RING) & 1, abort_flag, WAIT_LIMIT);
                            if (!ok) return;
                        }
                        if (h2 == 0) mbar_expect_tx(fb, C::UH * C::SLOT_BYTES);
                        uint8_t* dst = sSlot + (j % C::NSLOT) * C::SLOT_BYTES;
                        const int hf = un * C::UH + h2;
                        for (int c = 0; c < C::CH / C::EPB; c++)
                            tma_load_3d(dst + c * BOX_BYTES, map, fb, x0 + hf * C::CH + c * C::EPB, row, z);
                    }
                }
            };
            for (int n = 0; ok; n++) {
                int id = atomicAdd(p.sched + MODE, 1);
                if (id >= total) id = -1;
                item_ids[n & 3] = id;
                mbar_arrive(&bar_item[n & 3]);     // release: the id is visible to whoever passes the wait
                if (id < 0) break;
                const Item it = decode(id);
                // the stationary tile's buffer is free once the previous item's first contractions are done
                ok = mbar_wait<SLACK_SLEEP_NS>(bar_xfree, (n & 1) ^ 1, abort_flag, WAIT_LIMIT);
                if (!ok) break;
                mbar_expect_tx(bar_x, C::X_BYTES);
                for (int c = 0; c < DL / C::EPB; c++) {
                    if (MODE == STATE) tma_load_3d(sX + c * BOX_BYTES, &tmI, bar_x, c * C::EPB, it.half * TILE, 0);
                    else tma_load_3d(sX + c * BOX_BYTES, &tmX, bar_x, c * C::EPB, it.tile * TILE, it.bh);
                }
                auto load_y = [&](int t) {
                    if (is_state_step(t)) load_tile(&tmI, 0, t * TILE, 0);
                    else load_tile(&tmY, 0, stream_tile(it, t) * TILE, it.bh);
                };
                auto load_z = [&](int t) {
                    if (is_state_step(t)) load_tile(&tmS, 0, t * TILE, it.bh * p.NB + it.blk);
                    else load_tile(&tmZ, 0, stream_tile(it, t) * TILE, it.bh);
                };
                // same order as the MMA issuer consumes: Y(0), then Y(t), Z(t-1) ..., Z(last)
                load_y(0);
                for (int t = 1; t < it.nsteps && ok; t++) {
                    load_y(t);
                    load_z(t - 1);
                }
                if (ok) load_z(it.nsteps - 1);
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer
        // The whole warp runs this loop and one elected lane issues the MMAs and commits.  tcgen05.mma takes
        // its descriptors and addresses from warp-uniform registers: inside a one-lane branch the compiler
        // has to move every operand there instruction by instruction, and the issue of one MMA then costs
        // more cycles (about 100, measured) than a 128x128x16 MMA runs (64).  Kept convergent, with the
        // values that come out of memory passed through a shuffle from lane 0 so that they count as
        // uniform, the address arithmetic stays on the uniform datapath.
        {
            const bool issuer = elect_one();
            auto uni = [](int x) { return __shfl_sync(0xffffffffu, x, 0); };
            auto wait_u = [&](uint64_t* bar, uint32_t parity) { return mbar_wait_warp(bar, parity, abort_flag, WAIT_LIMIT); };
            constexpr uint32_t idesc1 = make_idesc(ABFMT, 128, 128, 0, 0);
            constexpr uint32_t idesc2 = make_idesc(ABFMT, 128, X3 ? D : C::CH, 0, 1);
            constexpr int KROWS_BYTES = C::KSTEP * 128;  // KSTEP streamed rows of the Z tile
            const uint32_t sX_u = static_cast<uint32_t>(uni(static_cast<int>(smem_u32(sX))));
            const uint32_t sSlot_u = sX_u + C::X_BYTES;
            const uint32_t tmem_T0u = static_cast<uint32_t>(uni(static_cast<int>(tmem_T0)));
            const uint32_t tmem_ACCu = tmem_T0u + 256;
            const uint64_t xdesc0 = smem_desc_sw128(sX_u, 16, 1024);           // K-major stationary tile
            const uint64_t ydesc0 = smem_desc_sw128(sSlot_u, 16, 1024);        // K-major view of slot 0
            const uint64_t zdesc0 = TF32 ? smem_desc_sw128(sSlot_u, BOX_BYTES, 512, 1)   // MN-major view of slot 0:
                                         : smem_desc_sw128(sSlot_u, BOX_BYTES, 1024, 2); // 32-bit tiles use the 32-byte-atom swizzle
            int useq = 0;      // units consumed so far
            int gstep = 0;     // steps issued by this CTA over all its items: T buffer and barrier phases follow it
            bool ok = true;
            for (int n = 0; ok; n++) {
                ok = wait_u(&bar_item[n & 3], (n >> 2) & 1);
                if (!ok) break;
                const int id = uni(item_ids[n & 3]);
                if (id < 0) break;
                const Item it = decode(id);
                ok = wait_u(bar_x, n & 1);
                if (!ok) break;
                tc_fence_after();
                // Between two MMAs the issuing lane has time to spare (the tensor pipe holds the issue back to its
                // own pace), between two batches it has none: whatever the warp does there leaves the pipe idle.
                // So the barriers the next batch depends on are tested in the middle of the current batch; at the
                // boundary a barrier is waited for only if that test failed.
                auto try_u = [&](uint64_t* bar, uint32_t parity) {
                    return __all_sync(0xffffffffu, mbar_test_wait(bar, parity) ? 1 : 0) != 0;
                };
                bool preY = false;   // "loaded" barrier of the next Y tile's first unit seen complete
                bool preW = false;   // W(t-1) seen complete (and the tcgen05 fence after it executed)
                bool preZ = false;   // "loaded" barrier of Z(t-1)'s first unit seen complete
                auto second = [&](int u) {  // ACC += W(u) Z(u)
                    const int gu = gstep + u;
                    if (!preW) {
                        ok = ok && wait_u(&bar_w[gu & 1], (gu >> 1) & 1);
                        if (ok) tc_fence_after();
                    }
                    // the accumulator must have been drained by the previous item's epilogue
                    if (ok && u == 0) {
                        ok = wait_u(bar_accfree, (n & 1) ^ 1);
                        if (ok) tc_fence_after();
                    }
                    if (!ok) return;
                    const uint32_t w_tmem = tmem_T0u + (gu & 1) * 128;
                    constexpr int KS2 = TILE / C::KSTEP;   // KSTEP streamed rows per MMA
                    preY = false;
#pragma unroll
                    for (int un = 0; un < C::UPT; un++, useq++) {
                        if (!(un == 0 && preZ)) ok = wait_u(&bar_full[useq % C::RING], (useq / C::RING) & 1);   // TMA data: no tcgen05 fence
                        if (!ok) return;
#pragma unroll
                        for (int part = 0; part < 2; part++) {
                            if constexpr (X3) {
                                if (issuer) {
#pragma unroll
                                    for (int pr = 0; pr < 3; pr++) {   // (W hi, Z hi), (W hi, Z mid), (W mid, Z hi)
                                        const int box = (pr == 1) ? NBX : 0;   // first box of the Z half
                                        const uint64_t zdesc = smem_desc_advance(
                                            zdesc0, ((useq * C::UH + box / BPS) % C::NSLOT) * C::SLOT_BYTES + (box % BPS) * BOX_BYTES);
#pragma unroll
                                        for (int kk = 0; kk < KS2; kk++) {
                                            if (((pr * KS2 + kk) * 2) / (3 * KS2) != part) continue;
                                            // W hi of gate group g in columns [32g, 32g+16), W mid in [32g+16, 32g+32)
                                            const uint32_t at = w_tmem + (kk >> 1) * 32 + (kk & 1) * 8 + (pr == 2 ? 16 : 0);
                                            mma_ts<false>(tmem_ACCu, at, smem_desc_advance(zdesc, kk * KROWS_BYTES), idesc2,
                                                          (u > 0 || pr > 0 || kk > 0) ? 1u : 0u);
                                        }
                                    }
                                    if (part == 1) tc_commit(&bar_cons[useq % C::RING]);
                                }
                            } else if (issuer) {
#pragma unroll
                                for (int h2 = 0; h2 < C::UH; h2++) {
                                    const int hf = un * C::UH + h2;
                                    const uint64_t zdesc = smem_desc_advance(zdesc0, ((useq * C::UH + h2) % C::NSLOT) * C::SLOT_BYTES);
#pragma unroll
                                    for (int kk = 0; kk < KS2; kk++) {
                                        if (((h2 * KS2 + kk) * 2) / (C::UH * KS2) != part) continue;
                                        // 16-bit W: gate group g packed streamed rows [32g, 32g+32) into columns
                                        // [32g, 32g+16); 32-bit W: row j in column j.  Either way a K step is 8 columns.
                                        const uint32_t at = TF32 ? (w_tmem + kk * 8) : (w_tmem + (kk >> 1) * 32 + (kk & 1) * 8);
                                        mma_ts<TF32>(tmem_ACCu + hf * C::CH, at, smem_desc_advance(zdesc, kk * KROWS_BYTES), idesc2,
                                                     (u > 0 || kk > 0) ? 1u : 0u);
                                    }
                                }
                                if (part == 1) tc_commit(&bar_cons[useq % C::RING]);
                            }
                            __syncwarp();
                            // next in line after this tile: Y(u + 2), if the item has one
                            if (part == 0 && un == C::UPT - 1 && u + 2 < it.nsteps)
                                preY = try_u(&bar_full[(useq + 1) % C::RING], ((useq + 1) / C::RING) & 1);
                        }
                    }
                };
                for (int t = 0; t < it.nsteps && ok; t++) {
                    // T(t) = X Y(t)^T
                    const int gt = gstep + t;
                    const uint32_t t_tmem = tmem_T0u + (gt & 1) * 128;
                    constexpr int KS1 = C::CH / C::KSTEP;
                    preW = false;
                    preZ = false;
#pragma unroll
                    for (int un = 0; un < C::UPT; un++, useq++) {
                        if (!(un == 0 && preY)) ok = wait_u(&bar_full[useq % C::RING], (useq / C::RING) & 1);
                        if (!ok) break;
#pragma unroll
                        for (int part = 0; part < 2; part++) {
                            if constexpr (X3) {
                                if (issuer) {
                                    constexpr int KSX = D / 16;    // K steps per operand half
#pragma unroll
                                    for (int pr = 0; pr < 3; pr++) {   // (X hi, Y hi), (X hi, Y mid), (X mid, Y hi)
#pragma unroll
                                        for (int ks = 0; ks < KSX; ks++) {
                                            if (((pr * KSX + ks) * 2) / (3 * KSX) != part) continue;
                                            const int xb = (pr == 2 ? NBX : 0) + (ks >> 2), yb = (pr == 1 ? NBX : 0) + (ks >> 2);
                                            const uint64_t yd = smem_desc_advance(
                                                ydesc0, ((useq * C::UH + yb / BPS) % C::NSLOT) * C::SLOT_BYTES + (yb % BPS) * BOX_BYTES + (ks & 3) * 32);
                                            mma_ss<false>(t_tmem, smem_desc_advance(xdesc0, xb * BOX_BYTES + (ks & 3) * 32), yd, idesc1,
                                                          (pr > 0 || ks > 0) ? 1u : 0u);
                                        }
                                    }
                                    if (part == 1) {
                                        tc_commit(&bar_cons[useq % C::RING]);
                                        if (t == it.nsteps - 1) tc_commit(bar_xfree);
                                    }
                                }
                            } else if (issuer) {
#pragma unroll
                                for (int h2 = 0; h2 < C::UH; h2++) {
                                    const int hf = un * C::UH + h2;
                                    const uint64_t ydesc = smem_desc_advance(ydesc0, ((useq * C::UH + h2) % C::NSLOT) * C::SLOT_BYTES);
#pragma unroll
                                    for (int kk = 0; kk < KS1; kk++) {
                                        if (((h2 * KS1 + kk) * 2) / (C::UH * KS1) != part) continue;
                                        const int kx = hf * KS1 + kk;  // K step inside the stationary tile; four (4 x 32 bytes) per box row
                                        mma_ss<TF32>(t_tmem, smem_desc_advance(xdesc0, (kx >> 2) * BOX_BYTES + (kx & 3) * 32),
                                                     smem_desc_advance(ydesc, (kk >> 2) * BOX_BYTES + (kk & 3) * 32), idesc1,
                                                     (hf > 0 || kk > 0) ? 1u : 0u);
                                    }
                                }
                                if (part == 1) {
                                    // the unit is consumed; for the tile's last unit this is also "T(t) written"
                                    tc_commit(&bar_cons[useq % C::RING]);
                                    if (un == C::UPT - 1 && t == it.nsteps - 1) tc_commit(bar_xfree);   // stationary tile read for the last time
                                }
                            }
                            __syncwarp();
                            if (part == 0 && un == C::UPT - 1 && t >= 1) {   // next in line: W(t-1), then Z(t-1)
                                const int gu = gt - 1;
                                preW = try_u(&bar_w[gu & 1], (gu >> 1) & 1);
                                if (preW) tc_fence_after();
                                preZ = try_u(&bar_full[(useq + 1) % C::RING], ((useq + 1) / C::RING) & 1);
                            }
                        }
                    }
                    preY = false;
                    if (!ok) break;
                    if (t >= 1) second(t - 1);
                }
                preW = false;
                preZ = false;
                if (ok) second(it.nsteps - 1);
                if (ok && issuer) tc_commit(bar_acc);
                __syncwarp();
                gstep += it.nsteps;
            }
        }
    } else {
        // ------------------------------------------------------------ gate groups
        const int grp = (warp - 2) >> 2;               // warps 2..17: four groups of four warps
        const int r = (warp & 3) * 32 + lane;          // TMEM lane == row inside the tile (lane quarter = warp % 4)
        const uint32_t lane_bits = static_cast<uint32_t>((warp & 3) * 32) << 16;
        // Every group works on every step: group g gates columns [32g, 32g+32) of the T tile and writes
        // its part of W over them.
        const int cbase = grp * 32;
        auto load_cols = [&](const float* base, float (&dst)[32]) {
            const float4* p4 = reinterpret_cast<const float4*>(base + cbase);
#pragma unroll
            for (int q4 = 0; q4 < 8; q4++) {
                const float4 e4 = __ldg(p4 + q4);
                dst[q4 * 4 + 0] = e4.x; dst[q4 * 4 + 1] = e4.y; dst[q4 * 4 + 2] = e4.z; dst[q4 * 4 + 3] = e4.w;
            }
        };
        bool ok = true;
        int gstep = 0;
        [[maybe_unused]] uint8_t* stage = sOut + (warp - 2) * C::STAGE_BYTES;
        if (STAGED && lane == 0) prefetch_tmap(&tmO);
        // Row terms of a work item: the row part of the exponent in double (the column block's reference is added
        // per block; STATE: rows are key dimensions and every row carries the block-end stabiliser), the weight of
        // the inbound-state step of FWDC (exp(A_prev_block_end - A_row) / sqrt(D); -inf when there is no carry)
        // and the additive term of DQ.  Fetching (the loads) and combining (the first use of what was loaded) are
        // separate steps: the next item's terms are requested before the accumulator wait of this item and combined
        // only when that item starts, so nobody waits for those loads.
        struct RowRaw {
            float rel, g;
            double ref, b0, b1, lb;
        };
        auto fetch_rows = [&](const Item& it) {
            RowRaw rr{0.0f, 0.0f, 0.0, 0.0, 0.0, static_cast<double>(INFINITY)};
            const int grow = it.tile * TILE + r;
            const size_t vec_base = static_cast<size_t>(it.bh) * p.Spad;
            if (CHUNKED || MODE == STATE) {
                const double* bound = p.An_bound + static_cast<size_t>(it.bh) * (p.NB + 1) + it.blk;
                rr.b0 = bound[0];
                rr.b1 = bound[1];
                if (MODE == FWDC && p.late_bound) rr.lb = p.late_bound[it.bh];
            }
            if (MODE != STATE) {
                rr.rel = p.row_rel[vec_base + grow];
                rr.ref = p.row_ref[static_cast<size_t>(it.bh) * (p.Spad / REF_BLOCK) + grow / REF_BLOCK];
            }
            if (IS_DQ) rr.g = p.row_g[vec_base + grow];
            return rr;
        };
        constexpr int UNKNOWN = -2;
        int id = next_item(0, ok);
        RowRaw raw{0.0f, 0.0f, 0.0, 0.0, 0.0, static_cast<double>(INFINITY)};
        if (ok && id >= 0) raw = fetch_rows(decode(id));

        for (int n = 0; ok && id >= 0; n++) {
        const Item it = decode(id);
        const int bh = it.bh, tile = it.tile, blk = it.blk, nsteps = it.nsteps;
        const int grow = tile * TILE + r;              // row inside the slice (may be >= S in the last tile)
        const size_t vec_base = static_cast<size_t>(bh) * p.Spad;
        const size_t ref_base = static_cast<size_t>(bh) * (p.Spad / REF_BLOCK);
        // FWDC with a late carry: the row's stabiliser -A*log2e and the inbound block boundary are capped by the
        // carried-in maximum, and m grows by what the cap took off
        const double negA = static_cast<double>(raw.rel) + raw.ref;
        const double negA_c = (MODE == FWDC) ? fmin(negA, raw.lb) : negA;
        const float m_shift = (MODE == FWDC) ? static_cast<float>((negA - negA_c) * 0.6931471805599453) : 0.0f;
        // STATE: every row carries the block's stabiliser: -A_end(block) for the forward states, +A_end(previous
        // block) for the states carried back in the backward (weights exp(A_end(k-1) - A_t) scale / n_t)
        const double er_d = (MODE == STATE) ? (p.state_reverse ? -raw.b0 : raw.b1) : negA_c + static_cast<double>(p.er_add);
        // log2 of the row weight of the state step: FWDC, DQC exp(A_end(k-1) - A_t) (times scale, resp. scale / n_t);
        // DKC, DVC exp(a_j - A_end(k))
        const float er_state = !CHUNKED ? 0.0f
                               : ROWS_ARE_Q ? static_cast<float>(er_d - fmin(raw.b0, raw.lb)) : static_cast<float>(er_d + raw.b1);
        const float state_w = (MODE == DQC || MODE == DKC) ? fast_exp2(er_state) : 0.0f;   // for the epilogue's rank-1 term
        const float g_row = raw.g;
        float rowsum = 0.0f;

        for (int t = 0; t < nsteps; t++) {
            const int gt = gstep + t;
            const int buf = gt & 1;
            const bool state_step = is_state_step(t);
            const int st = state_step ? 0 : stream_tile(it, t);
            const bool diag = (MODE != STATE) && !state_step && (st == tile);
            // On the diagonal tile the 32 x 32 patch of a gate group and a row quarter lies wholly on the masked side
            // for six of the sixteen (group, quarter) pairs: those warps write zeros over their part of T and read nothing.
            if (diag && (ROWS_ARE_Q ? (grp > (warp & 3)) : (grp < (warp & 3)))) {
                const int sq0 = (2 * gstep + (t == 0 ? 0 : 2 * t - 1) + 1) * C::UPT - 1;
                ok = mbar_wait_warp<SLACK_SLEEP_NS>(&bar_cons[sq0 % C::RING], (sq0 / C::RING) & 1, abort_flag, WAIT_LIMIT);
                if (!ok) break;
                tc_fence_after();
                const uint32_t z_tmem = tmem_T0 + buf * 128 + lane_bits + cbase;
                if constexpr (TF32 || X3) {
                    uint32_t zv[32];
#pragma unroll
                    for (int j = 0; j < 32; j++) zv[j] = 0u;
                    tmem_st32(z_tmem, zv);
                } else {
                    uint32_t zv[16];
#pragma unroll
                    for (int j = 0; j < 16; j++) zv[j] = 0u;
                    tmem_st16(z_tmem, zv);
                }
                tc_wait_st();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(&bar_w[buf]);
                continue;
            }
            // state step: the column term is the inbound normaliser vector z (a weight, not an exponent)
            // off the diagonal the column term comes as a factor exp2(ec) (see gates.cu), on the diagonal tile as
            // the exponent itself: there a masked column can lie above the row's maximum and only the sum is safe
            const float* ce = (state_step && MODE == FWDC) ? p.zstate + (static_cast<size_t>(bh) * p.NB + blk) * D + t * TILE
                                                           : (diag ? p.col_rel : p.col_w) + vec_base + st * TILE;
            // column terms do not depend on the contraction: fetch them before waiting
            float cv[32];
            load_cols(ce, cv);
            const float er = state_step ? er_state
                                        : static_cast<float>(er_d + p.col_ref[ref_base + st * (TILE / REF_BLOCK) + (grp >> 1)]);
            const float er_w = (CHUNKED && state_step) ? fast_exp2(er) : 0.0f;
            // DK adds a per-column term to T.  Each lane fetches one column's value before the wait (32 more
            // registers are not to be had) and the warp passes them round with shuffles afterwards.
            const float g_lane = (IS_DK && !state_step) ? __ldg(p.col_g + vec_base + st * TILE + cbase + lane) : 0.0f;
            // units before the last one of Y(t): tiles go Y(0), Y(1), Z(0), Y(2), Z(1), ... in every item
            const int sq = (2 * gstep + (t == 0 ? 0 : 2 * t - 1) + 1) * C::UPT - 1;
            ok = mbar_wait_warp<SLACK_SLEEP_NS>(&bar_cons[sq % C::RING], (sq / C::RING) & 1, abort_flag, WAIT_LIMIT);
            if (!ok) break;
            tc_fence_after();
            const uint32_t t_tmem = tmem_T0 + buf * 128 + lane_bits + cbase;
            uint32_t tv[32];
            tmem_ld32(t_tmem, tv);
            tc_wait_ld();
            if (IS_DK && !state_step) {   // T + g with g per column: added eight columns at a time to keep registers free
#pragma unroll
                for (int j = 0; j < 32; j++)
                    tv[j] = __float_as_uint(__uint_as_float(tv[j]) + __shfl_sync(0xffffffffu, g_lane, j));
            }
            if (CHUNKED && state_step) {
#pragma unroll
                for (int j = 0; j < 32; j++) {
                    const float wj = __uint_as_float(tv[j]) * er_w;   // T = X: scale the row; FWDC: b += (scaled q) . z
                    if (MODE == FWDC) rowsum = fmaf(wj, cv[j], rowsum);
                    cv[j] = wj;
                }
            } else if (diag) {
#pragma unroll
                for (int j = 0; j < 32; j++) {
                    float tval = __uint_as_float(tv[j]);
                    if (IS_DQ) tval += g_row;
                    float wj = tval * fast_exp2(cv[j] + er);
                    if (!causal_ok<MODE>(r, cbase + j)) wj = 0.0f;
                    if (IS_FWD) rowsum += wj;
                    cv[j] = wj;
                }
            } else {
                // exp2(ec + er) = exp2(ec) exp2(er): one exponential per row and step; both factors are <= const
                // because every column of an off-diagonal tile is on the causal side of every row
                // A 64-column block that is padding from end to end (ragged S) has no meaningful reference, and the
                // row term alone can be large with strong decay: its column factors are 0, and 0 times an overflowed
                // u would be NaN.  Real columns keep er far below the clamp.
                const float u = fast_exp2(fminf(er, MAX_ROW_EXP2));
                const float gu = IS_DQ ? g_row * u : 0.0f;
#pragma unroll
                for (int j = 0; j < 32; j++) {
                    const float tu = IS_DQ ? fmaf(__uint_as_float(tv[j]), u, gu) : __uint_as_float(tv[j]) * u;
                    const float wj = tu * cv[j];
                    if (IS_FWD || MODE == STATE) rowsum += wj;
                    cv[j] = wj;
                }
            }
            if constexpr (TF32) {
#pragma unroll
                for (int j = 0; j < 32; j++) tv[j] = to_tf32(cv[j]);
                tmem_st32(t_tmem, tv);   // in place: column for column
            } else if constexpr (X3) {
#pragma unroll
                for (int j = 0; j < 16; j++) {   // W = hi + mid, both bf16: hi halves in the first 16 columns, mid in the other 16
                    __nv_bfloat162 hi2 = __floats2bfloat162_rn(cv[2 * j], cv[2 * j + 1]);
                    const float2 hf2 = __bfloat1622float2(hi2);
                    __nv_bfloat162 mid2 = __floats2bfloat162_rn(cv[2 * j] - hf2.x, cv[2 * j + 1] - hf2.y);
                    tv[j] = *reinterpret_cast<uint32_t*>(&hi2);
                    tv[16 + j] = *reinterpret_cast<uint32_t*>(&mid2);
                }
                tmem_st32(t_tmem, tv);
            } else {
                uint32_t pk[16];
#pragma unroll
                for (int j = 0; j < 16; j++) {
                    if constexpr (ABFMT == 1) {
                        __nv_bfloat162 v2 = __floats2bfloat162_rn(cv[2 * j], cv[2 * j + 1]);
                        pk[j] = *reinterpret_cast<uint32_t*>(&v2);
                    } else {
                        __half2 v2 = __floats2half2_rn(cv[2 * j], cv[2 * j + 1]);
                        pk[j] = *reinterpret_cast<uint32_t*>(&v2);
                    }
                }
                tmem_st16(t_tmem, pk);   // two values per column, over the first 16 of this group's 32 columns
            }
            tc_wait_st();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&bar_w[buf]);   // 16 arrivals instead of 512 on one shared-memory word
        }
        if (!ok) break;
        gstep += nsteps;

        // ---- while the last contractions run: everything of the epilogue that does not need the accumulator
        constexpr int QUART = D / NGROUPS;             // 16, 32 or 64 columns
        constexpr int CW = QUART < 32 ? QUART : 32;    // columns per TMEM load
        constexpr int VEC = 16 / sizeof(SideT);        // elements per 16-byte access of the tensors read in the epilogue
        const int c0 = grp * QUART;
        const bool row_ok = (MODE == STATE) ? true : (grow < p.S);
        float* part = part_base + (C::PARTS == 2 ? (n & 1) * NGROUPS * 128 : 0);
        float inv_n = 1.0f;
        auto exchange = [&](float x) {   // sum of one value per gate group for this row (once per item)
            part[grp * 128 + r] = x;
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_part);
            ok = mbar_wait_warp<SLACK_SLEEP_NS>(bar_part, n & 1, abort_flag, WAIT_LIMIT);
            return ok ? (part[r] + part[128 + r]) + (part[256 + r] + part[384 + r]) : 0.0f;
        };
        auto row_sums = [&]() {
            if (MODE == STATE) {
                const float zsum = exchange(rowsum);
                if (ok && grp == 0 && p.b_out) p.b_out[(static_cast<size_t>(bh) * p.NB + blk) * D + it.half * TILE + r] = zsum;
            }
            if (IS_FWD) {
                // on its way during the exchange
                const float mrow = row_ok ? p.m[static_cast<size_t>(bh) * p.S + grow] + m_shift : 0.0f;
                const float bsum = exchange(rowsum);
                if (ok) {
                    const float nrm = fmaxf(fabsf(bsum), __expf(-mrow)) + 1e-6f;
                    inv_n = 1.0f / nrm;
                    if (grp == 0 && row_ok && p.b_out) p.b_out[static_cast<size_t>(bh) * p.S + grow] = bsum;
                }
            }
        };
        // When may the row partials be written?  Once nobody reads the ones written two items ago (alternating
        // buffers) resp. by the previous item (one buffer).  A warp is past this item's gate steps only after the
        // previous item's accumulator was complete, i.e. after every warp had done that item's gate steps and with
        // them its epilogue before: two items back is always safe.  With one buffer it is safe here only if this
        // item has more than two steps (the third T tile follows the first W tile, which needs every warp), else
        // after the accumulator wait (which needs every warp's last W tile of this item).
        const bool sums_early = (C::PARTS == 2) || nsteps > 2;
        if (sums_early) row_sums();
        if (!ok) break;
        // next work item, if it is published already, and its row terms
        int id_next = UNKNOWN;
        RowRaw raw_next{0.0f, 0.0f, 0.0, 0.0, 0.0, static_cast<double>(INFINITY)};
        if (__all_sync(0xffffffffu, mbar_test_wait(&bar_item[(n + 1) & 3], ((n + 1) >> 2) & 1) ? 1 : 0)) {
            id_next = __shfl_sync(0xffffffffu, item_ids[(n + 1) & 3], 0);
            if (id_next >= 0) raw_next = fetch_rows(decode(id_next));
        }

        // ---- epilogue: each group drains a quarter of the accumulator's columns for all 128 rows
        ok = mbar_wait_warp<SLACK_SLEEP_NS>(bar_acc, n & 1, abort_flag, WAIT_LIMIT);
        if (!ok) break;
        {
            tc_fence_after();
            if (!sums_early) row_sums();
            if (!ok) break;
            // STATE writes block (bh, blk) of [BH, NB, D, D]; everything else row `grow` of [BH, S, D]
            const size_t row_off = (MODE == STATE)
                                       ? ((static_cast<size_t>(bh) * p.NB + blk) * D + it.half * TILE + r) * D
                                       : (static_cast<size_t>(bh) * p.S + (row_ok ? grow : 0)) * D;
            float dot = 0.0f;
            OutT* orow = reinterpret_cast<OutT*>(p.out) + row_off + c0;
            const SideT* ogate_row = (IS_FWD && p.ogate) ? reinterpret_cast<const SideT*>(p.ogate) + row_off + c0 : nullptr;
            const SideT* drow = ((IS_DQ || IS_DK) && p.dot_src)
                                    ? reinterpret_cast<const SideT*>(p.dot_src) + row_off + c0 : nullptr;
            // DQC / DKC: the state step leaves out a rank-1 term, coef_row * vec[column]:
            //   dQ_t += beta_t g_t z_k    (the db part of the carried-in state, z_k the inbound normaliser vector)
            //   dK_j += gamma_j r_k       (r_k: the same part of the state carried back from the later blocks)
            [[maybe_unused]] const float rank1_coef = (MODE == DQC) ? state_w * g_row : state_w;
            [[maybe_unused]] const float* rank1_vec = (MODE == DQC || MODE == DKC)
                                         ? (MODE == DQC ? p.zstate : p.rvec) + (static_cast<size_t>(bh) * p.NB + blk) * D + c0 : nullptr;
#pragma unroll 1
            for (int ch = 0; ch < QUART / CW; ch++) {
                uint32_t av[32];
                if constexpr (CW == 32) {
                    tmem_ld32(tmem_ACC + lane_bits + c0 + ch * 32, av);
                } else {
                    tmem_ld16(tmem_ACC + lane_bits + c0, reinterpret_cast<uint32_t (&)[16]>(av));
                }
                tc_wait_ld();
                if (ch == QUART / CW - 1) {
                    // this warp's share of the accumulator is in registers: the next item may overwrite it
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(bar_accfree);
                }
                float vals[CW];
#pragma unroll
                for (int j = 0; j < CW; j++) vals[j] = __uint_as_float(av[j]) * inv_n;
                if constexpr (MODE == DQC || MODE == DKC) {
#pragma unroll
                    for (int j4 = 0; j4 < CW / 4; j4++) {
                        const float4 e4 = __ldg(reinterpret_cast<const float4*>(rank1_vec + ch * CW) + j4);
                        vals[j4 * 4 + 0] = fmaf(rank1_coef, e4.x, vals[j4 * 4 + 0]);
                        vals[j4 * 4 + 1] = fmaf(rank1_coef, e4.y, vals[j4 * 4 + 1]);
                        vals[j4 * 4 + 2] = fmaf(rank1_coef, e4.z, vals[j4 * 4 + 2]);
                        vals[j4 * 4 + 3] = fmaf(rank1_coef, e4.w, vals[j4 * 4 + 3]);
                    }
                }
                if (row_ok) {
                    if (IS_FWD && ogate_row) {
#pragma unroll
                        for (int j = 0; j < CW; j++) vals[j] *= silu_f(to_f32<SideT>(ogate_row[ch * CW + j]));
                    }
                    if ((IS_DQ || IS_DK) && drow) {
#pragma unroll
                        for (int jv = 0; jv < CW / VEC; jv++) {
                            const uint4 raw = *reinterpret_cast<const uint4*>(drow + ch * CW + jv * VEC);
                            const SideT* ev = reinterpret_cast<const SideT*>(&raw);
#pragma unroll
                            for (int j = 0; j < VEC; j++) dot += vals[jv * VEC + j] * to_f32<SideT>(ev[j]);
                        }
                    }
                }
                if constexpr (STAGED) {
                    // This warp's 32 rows x 32 columns go out through its staging buffer (64-byte swizzle: no bank
                    // conflicts) and a TMA store; rows past the end of the tensor are not written.  Scattered
                    // stores from registers, one row per thread, keep the gate warps busy for thousands of cycles
                    // per item, during which the tensor pipe has nothing to do.
                    static_assert(CW == 32, "staged output is built for 32-column chunks");
                    constexpr int NSUB = sizeof(OutT) == 4 ? 2 : 1;    // 64 bytes per row and store
#pragma unroll
                    for (int sub = 0; sub < NSUB; sub++) {
                        if (lane == 0) bulk_wait_read_all();   // the previous store has read the buffer
                        __syncwarp();
                        uint4* srow = reinterpret_cast<uint4*>(stage + lane * 64);
                        const int sw = (lane >> 1) & 3;
                        if constexpr (sizeof(OutT) == 4) {
#pragma unroll
                            for (int j4 = 0; j4 < 4; j4++)
                                srow[j4 ^ sw] = make_uint4(__float_as_uint(vals[sub * 16 + j4 * 4]), __float_as_uint(vals[sub * 16 + j4 * 4 + 1]),
                                                           __float_as_uint(vals[sub * 16 + j4 * 4 + 2]), __float_as_uint(vals[sub * 16 + j4 * 4 + 3]));
                        } else {
#pragma unroll
                            for (int j4 = 0; j4 < 4; j4++) {
                                uint32_t o32[4];
#pragma unroll
                                for (int j = 0; j < 4; j++) {   // two values per conversion
                                    if constexpr (ABFMT == 1) {
                                        __nv_bfloat162 v2 = __floats2bfloat162_rn(vals[j4 * 8 + 2 * j], vals[j4 * 8 + 2 * j + 1]);
                                        o32[j] = *reinterpret_cast<uint32_t*>(&v2);
                                    } else {
                                        __half2 v2 = __floats2half2_rn(vals[j4 * 8 + 2 * j], vals[j4 * 8 + 2 * j + 1]);
                                        o32[j] = *reinterpret_cast<uint32_t*>(&v2);
                                    }
                                }
                                srow[j4 ^ sw] = make_uint4(o32[0], o32[1], o32[2], o32[3]);
                            }
                        }
                        fence_async_smem();
                        __syncwarp();
                        if (lane == 0) {
                            const int x = c0 + ch * 32 + sub * (64 / static_cast<int>(sizeof(OutT)));
                            if (MODE == STATE) tma_store_3d(&tmO, stage, x, (warp & 3) * 32, bh * p.NB + blk);
                            else tma_store_3d(&tmO, stage, x, tile * TILE + (warp & 3) * 32, bh);
                            bulk_commit();
                        }
                    }
                } else if (row_ok) {
                    if constexpr (sizeof(OutT) == 4) {
#pragma unroll
                        for (int j4 = 0; j4 < CW / 4; j4++) {
                            float4 o4 = make_float4(vals[j4 * 4], vals[j4 * 4 + 1], vals[j4 * 4 + 2], vals[j4 * 4 + 3]);
                            *reinterpret_cast<float4*>(reinterpret_cast<float*>(orow) + ch * CW + j4 * 4) = o4;
                        }
                    } else {
#pragma unroll
                        for (int j8 = 0; j8 < CW / 8; j8++) {
                            uint4 o4;
                            uint32_t* o32 = reinterpret_cast<uint32_t*>(&o4);
#pragma unroll
                            for (int j = 0; j < 4; j++) {
                                OutT lo = from_f32<OutT>(vals[j8 * 8 + 2 * j]);
                                OutT hi = from_f32<OutT>(vals[j8 * 8 + 2 * j + 1]);
                                o32[j] = static_cast<uint32_t>(*reinterpret_cast<uint16_t*>(&lo)) |
                                         (static_cast<uint32_t>(*reinterpret_cast<uint16_t*>(&hi)) << 16);
                            }
                            *reinterpret_cast<uint4*>(orow + ch * CW + j8 * 8) = o4;
                        }
                    }
                }
            }
            // one partial per gate group: adding them up is left to the dF kernel, so that the groups need not meet here
            if ((IS_DQ || IS_DK) && p.dot_out) p.dot_out[grp * p.dot_part_stride + vec_base + grow] = row_ok ? dot : 0.0f;
        }
        if (!ok) break;
        // ---- on to the next item
        if (id_next == UNKNOWN) {
            id_next = next_item(n + 1, ok);
            if (ok && id_next >= 0) raw_next = fetch_rows(decode(id_next));
        }
        id = id_next;
        raw = raw_next;
        }  // items
        if (STAGED && lane == 0) bulk_wait_all();   // the last stores have left shared memory before the CTA goes away
        tc_fence_before();
    }

    __syncthreads();
    if (*abort_flag) {
        if (threadIdx.x == 0) atomicExch(p.status, 1000 + MODE);
        // give copies and MMAs that are still in flight time to land before the CTA's memory goes away
        for (int k = 0; k < 64; k++) __nanosleep(16000);
        __syncthreads();
    }
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, 512);
    }
}

// ------------------------------------------------------------------ host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode() {
    static std::atomic<EncodeTiledFn> fn{nullptr};   // the lookup is idempotent: concurrent first callers agree
    EncodeTiledFn f = fn.load(std::memory_order_acquire);
    if (f) return f;
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres) != cudaSuccess ||
        qres != cudaDriverEntryPointSuccess)
        return nullptr;
    f = reinterpret_cast<EncodeTiledFn>(sym);
    fn.store(f, std::memory_order_release);
    return f;
}

// Encoding a tensor map costs about a microsecond of host time, and one call of the library needs the same
// few maps in several passes: each host thread keeps the last maps it encoded, keyed by everything that goes in.
struct MapKey {
    const void* base;
    int n2, n1, n0, dtype, swizzle, box_rows, box_bytes, box_groups;
    bool operator==(const MapKey& o) const {
        return base == o.base && n2 == o.n2 && n1 == o.n1 && n0 == o.n0 && dtype == o.dtype && swizzle == o.swizzle &&
               box_rows == o.box_rows && box_bytes == o.box_bytes && box_groups == o.box_groups;
    }
};
struct MapCache {
    static constexpr int N = 32;
    MapKey keys[N] = {};
    CUtensorMap maps[N];
    bool used[N] = {};
    int next = 0;
    const CUtensorMap* find(const MapKey& k) const {
        for (int i = 0; i < N; i++)
            if (used[i] && keys[i] == k) return &maps[i];
        return nullptr;
    }
    void put(const MapKey& k, const CUtensorMap& m) {
        keys[next] = k; maps[next] = m; used[next] = true;
        next = (next + 1) % N;
    }
};
thread_local MapCache g_map_cache;

// [N2, N1, N0] tensor (N0 contiguous): boxes of box_bytes x box_rows, given swizzle, zero fill outside the tensor
int encode_map(CUtensorMap* map, const void* base, int N2, int N1, int N0, int dtype, CUtensorMapSwizzle swz, int box_rows,
               int box_bytes, CUtensorMapL2promotion promo) {
    const MapKey key{base, N2, N1, N0, dtype, static_cast<int>(swz), box_rows, box_bytes, 0};
    if (const CUtensorMap* hit = g_map_cache.find(key)) {
        *map = *hit;
        return MLSTM_OK;
    }
    EncodeTiledFn enc = get_encode();
    if (!enc) return MLSTM_E_CUDA;
    const cuuint64_t es = dtype == MLSTM_DT_F32 ? 4 : 2;
    cuuint64_t dims[3] = {static_cast<cuuint64_t>(N0), static_cast<cuuint64_t>(N1), static_cast<cuuint64_t>(N2)};
    cuuint64_t strides[2] = {static_cast<cuuint64_t>(N0) * es, static_cast<cuuint64_t>(N1) * N0 * es};
    cuuint32_t box[3] = {static_cast<cuuint32_t>(box_bytes / es), static_cast<cuuint32_t>(box_rows), 1};
    cuuint32_t estr[3] = {1, 1, 1};
    CUtensorMapDataType dt = dtype == MLSTM_DT_F32    ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                             : dtype == MLSTM_DT_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                                      : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    CUresult r = enc(map, dt, 3, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swz, promo,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return MLSTM_E_CUDA;
    g_map_cache.put(key, *map);
    return MLSTM_OK;
}

// Boxes of 128 bytes x box_rows rows with the 128-byte swizzle.
// atom32: 128-byte swizzle with 32-byte atoms (needed where a 32-bit tile is read MN-major).
int make_map(CUtensorMap* map, const void* base, int N2, int N1, int N0, int dtype, bool atom32 = false, int box_rows = 128) {
    return encode_map(map, base, N2, N1, N0, dtype, atom32 ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : CU_TENSOR_MAP_SWIZZLE_128B,
                      box_rows, 128, CU_TENSOR_MAP_L2_PROMOTION_L2_256B);
}

int sm_count() {
    static std::atomic<int> cached[MAX_DEVICES];   // zero-initialised; the query is idempotent
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= MAX_DEVICES) return -1;
    int n = cached[dev].load(std::memory_order_relaxed);
    if (n == 0) {
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return -1;
        cached[dev].store(n, std::memory_order_relaxed);
    }
    return n;
}

template <int MODE, int D, int ABFMT, typename OutT, bool X3 = false>
int launch_one(const PassParams& p_in, int in_dtype, cudaStream_t st) {
    PassParams p = p_in;
    p.slice_set = SLICE_SET_DEFAULT;
    CUtensorMap mx, my, mz, mi, ms, mo;
    int rc;
    constexpr int DL = X3 ? 2 * D : D;   // X3: X, Y, Z are the split copies, rows of hi | mid
    if ((rc = make_map(&mx, p.X, p.BH, p.S, DL, in_dtype)) != MLSTM_OK) return rc;
    if ((rc = make_map(&my, p.Y, p.BH, p.S, DL, in_dtype)) != MLSTM_OK) return rc;
    if ((rc = make_map(&mz, p.Z, p.BH, p.S, DL, in_dtype, ABFMT == 2)) != MLSTM_OK) return rc;
    mi = mx;
    ms = mx;
    constexpr bool CHUNKED = (MODE == FWDC || MODE == DQC || MODE == DKC || MODE == DVC);
    if (CHUNKED || MODE == STATE) {
        if (!p.ident || p.chunk_tiles <= 0 || p.NB <= 0 || !p.An_bound) return MLSTM_E_ARG;
        if ((rc = make_map(&mi, p.ident, 1, D, D, in_dtype)) != MLSTM_OK) return rc;
    }
    if (CHUNKED) {
        if (!p.states || ((MODE == FWDC || MODE == DQC) && !p.zstate) || (MODE == DKC && !p.rvec)) return MLSTM_E_ARG;
        if ((rc = make_map(&ms, p.states, p.BH * p.NB, D, D, in_dtype)) != MLSTM_OK) return rc;
    }
    mo = mx;
    if (TcCfg<DL, ABFMT == 2 ? 4 : 2>::STAGED && !X3) {
        constexpr int out_dtype = sizeof(OutT) == 4 ? MLSTM_DT_F32 : (ABFMT == 1 ? MLSTM_DT_BF16 : MLSTM_DT_F16);
        if (MODE == STATE) rc = tc_make_map_out(&mo, p.out, p.BH * p.NB, D, D, out_dtype, 32);
        else rc = tc_make_map_out(&mo, p.out, p.BH, p.S, D, out_dtype, 32);
        if (rc != MLSTM_OK) return rc;
    }
    auto kern = mlstm_tc_pass<MODE, D, ABFMT, OutT, X3>;
    constexpr int smem = TcCfg<DL, ABFMT == 2 ? 4 : 2>::SMEM_BYTES;
    cudaError_t ce;
    {   // the shared-memory opt-in is a per-device property of the kernel: set once per device
        static std::atomic<bool> opted[MAX_DEVICES];
        int dev = 0;
        if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= MAX_DEVICES) return MLSTM_E_CUDA;
        if (!opted[dev].load(std::memory_order_acquire)) {
            ce = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
            if (ce != cudaSuccess) {
                cudaGetLastError();
                return note_cuda_error(ce, "cudaFuncSetAttribute(MaxDynamicSharedMemorySize)");
            }
            opted[dev].store(true, std::memory_order_release);
        }
    }
    const int NT = p.Spad / TILE;
    const long long total = static_cast<long long>(MODE == STATE ? p.NB * (D / TILE) : NT) * p.BH;
    if (total > 0x7fffffffLL) return MLSTM_E_SHAPE;
    const int sms = sm_count();
    if (sms <= 0) return MLSTM_E_CUDA;
    const unsigned grid = static_cast<unsigned>(total < sms ? total : sms);  // persistent: one CTA per SM
    if (!p.sched) return MLSTM_E_ARG;
    if (!p.sched_zeroed) {
        ce = cudaMemsetAsync(p.sched + MODE, 0, sizeof(int), st);  // this pass's item counter
        if (ce != cudaSuccess) return note_cuda_error(ce, "cudaMemsetAsync(item counter)");
    }
    ce = launch_pdl(kern, dim3(grid), dim3(NTHREADS), smem, st, mx, my, mz, mi, ms, mo, p);
    if (ce != cudaSuccess) cudaGetLastError();
    return ce == cudaSuccess ? MLSTM_OK : note_cuda_error(ce, "launch of mlstm_tc_pass");
}

template <int MODE, int D, int ABFMT>
int launch_out(const PassParams& p, int in_dtype, int out_dtype, cudaStream_t st) {
    if (out_dtype == MLSTM_DT_F32) return launch_one<MODE, D, ABFMT, float>(p, in_dtype, st);
    if constexpr (ABFMT != 2) {
        if (out_dtype == in_dtype) {
            if (ABFMT == 1) return launch_one<MODE, D, ABFMT, __nv_bfloat16>(p, in_dtype, st);
            return launch_one<MODE, D, ABFMT, __half>(p, in_dtype, st);
        }
    }
    return MLSTM_E_ARG;
}

template <int MODE, int D>
int launch_fmt(const PassParams& p, int in_dtype, int out_dtype, cudaStream_t st) {
    if (in_dtype == MLSTM_DT_BF16) return launch_out<MODE, D, 1>(p, in_dtype, out_dtype, st);
    if (in_dtype == MLSTM_DT_F16) return launch_out<MODE, D, 0>(p, in_dtype, out_dtype, st);
    if constexpr (MODE <= DV) {
        if (in_dtype == MLSTM_DT_F32) return launch_out<MODE, D, 2>(p, in_dtype, out_dtype, st);
    }
    return MLSTM_E_UNSUPPORTED;
}

template <int MODE>
int launch_d(const PassParams& p, int in_dtype, int out_dtype, cudaStream_t st) {
    switch (p.D) {
        case 64: return launch_fmt<MODE, 64>(p, in_dtype, out_dtype, st);
        case 128: return launch_fmt<MODE, 128>(p, in_dtype, out_dtype, st);
        case 256: return launch_fmt<MODE, 256>(p, in_dtype, out_dtype, st);
    }
    return MLSTM_E_UNSUPPORTED;
}

}  // namespace


int tc_make_map(CUtensorMap* map, const void* base, int N2, int N1, int N0, int dtype, bool atom32, int box_rows) {
    return make_map(map, base, N2, N1, N0, dtype, atom32, box_rows);
}

int tc_make_map_out(CUtensorMap* map, const void* base, int N2, int N1, int N0, int dtype, int box_rows) {
    return encode_map(map, base, N2, N1, N0, dtype, CU_TENSOR_MAP_SWIZZLE_64B, box_rows, 64, CU_TENSOR_MAP_L2_PROMOTION_NONE);
}

// The same [N2, N1, N0] tensor seen as [N2, N0 / G, N1, G] with G = 128 bytes of elements: one box covers box_rows rows
// of box_groups neighbouring 128-byte column groups and lands in shared memory group after group (each group a
// box_rows x 128-byte block, 128-byte swizzled).  That is the layout of an MN-major MMA operand that is several
// column groups wide, fetched with ONE copy instead of one per group.  Coordinates: {0, row, group, slice}.
int tc_make_map_groups(CUtensorMap* map, const void* base, int N2, int N1, int N0, int dtype, bool atom32, int box_rows,
                       int box_groups) {
    const CUtensorMapSwizzle swz = atom32 ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : CU_TENSOR_MAP_SWIZZLE_128B;
    const MapKey key{base, N2, N1, N0, dtype, static_cast<int>(swz), box_rows, 128, box_groups};
    if (const CUtensorMap* hit = g_map_cache.find(key)) {
        *map = *hit;
        return MLSTM_OK;
    }
    EncodeTiledFn enc = get_encode();
    if (!enc) return MLSTM_E_CUDA;
    const cuuint64_t es = dtype == MLSTM_DT_F32 ? 4 : 2;
    const cuuint64_t G = 128 / es;
    if (N0 % static_cast<int>(G) != 0) return MLSTM_E_SHAPE;
    cuuint64_t dims[4] = {G, static_cast<cuuint64_t>(N1), static_cast<cuuint64_t>(N0) / G, static_cast<cuuint64_t>(N2)};
    cuuint64_t strides[3] = {static_cast<cuuint64_t>(N0) * es, 128, static_cast<cuuint64_t>(N1) * N0 * es};
    cuuint32_t box[4] = {static_cast<cuuint32_t>(G), static_cast<cuuint32_t>(box_rows), static_cast<cuuint32_t>(box_groups), 1};
    cuuint32_t estr[4] = {1, 1, 1, 1};
    CUtensorMapDataType dt = dtype == MLSTM_DT_F32    ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                             : dtype == MLSTM_DT_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                                      : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    CUresult r = enc(map, dt, 4, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swz,
                     CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return MLSTM_E_CUDA;
    g_map_cache.put(key, *map);
    return MLSTM_OK;
}

int tc_sm_count() { return sm_count(); }

int tc_slice_set() { return SLICE_SET_DEFAULT; }

bool tc_supported(int S, int D, int in_dtype) {
    return S >= 1 && (D == 64 || D == 128 || D == 256) &&
           (in_dtype == MLSTM_DT_F16 || in_dtype == MLSTM_DT_BF16 || in_dtype == MLSTM_DT_F32);
}

bool tc_x3_supported(int S, int D) { return S >= 1 && (D == 64 || D == 128); }

// fp32 problem on the tensor cores with split operands: p.X, p.Y, p.Z point to the bf16 hi | mid copies
// ([BH, S, 2 D]); everything else (outputs, dot_src, ogate) is fp32.
int launch_pass_tc_x3(int mode, const PassParams& p, cudaStream_t st) {
    if (!tc_x3_supported(p.S, p.D)) return MLSTM_E_UNSUPPORTED;
#define X3_CASE(M)                                                                             \
    case M:                                                                                    \
        return p.D == 64 ? launch_one<M, 64, 1, float, true>(p, MLSTM_DT_BF16, st)            \
                         : launch_one<M, 128, 1, float, true>(p, MLSTM_DT_BF16, st);
    switch (mode) {
        X3_CASE(FWD)
        X3_CASE(DQ)
        X3_CASE(DK)
        X3_CASE(DV)
    }
#undef X3_CASE
    return MLSTM_E_ARG;
}

int launch_pass_tc(int mode, const PassParams& p, int in_dtype, int out_dtype, cudaStream_t st) {
    if (!tc_supported(p.S, p.D, in_dtype)) return MLSTM_E_UNSUPPORTED;
    if (mode <= DV && tc_pair_supported(p.S, p.D, in_dtype)) return launch_pass_tc_pair(mode, p, in_dtype, out_dtype, st);
    switch (mode) {
        case FWD: return launch_d<FWD>(p, in_dtype, out_dtype, st);
        case DQ: return launch_d<DQ>(p, in_dtype, out_dtype, st);
        case DK: return launch_d<DK>(p, in_dtype, out_dtype, st);
        case DV: return launch_d<DV>(p, in_dtype, out_dtype, st);
        case FWDC:
            if (p.D == 256) return launch_fmt<FWDC, 256>(p, in_dtype, out_dtype, st);
            if (p.D != 128) return MLSTM_E_UNSUPPORTED;
            return launch_fmt<FWDC, 128>(p, in_dtype, out_dtype, st);
        case STATE:
            if (p.D == 256) return launch_fmt<STATE, 256>(p, in_dtype, out_dtype, st);
            if (p.D != 128) return MLSTM_E_UNSUPPORTED;
            return launch_fmt<STATE, 128>(p, in_dtype, out_dtype, st);
        case DQC:
            if (p.D == 256) return launch_fmt<DQC, 256>(p, in_dtype, out_dtype, st);
            if (p.D != 128) return MLSTM_E_UNSUPPORTED;
            return launch_fmt<DQC, 128>(p, in_dtype, out_dtype, st);
        case DKC:
            if (p.D == 256) return launch_fmt<DKC, 256>(p, in_dtype, out_dtype, st);
            if (p.D != 128) return MLSTM_E_UNSUPPORTED;
            return launch_fmt<DKC, 128>(p, in_dtype, out_dtype, st);
        case DVC:
            if (p.D == 256) return launch_fmt<DVC, 256>(p, in_dtype, out_dtype, st);
            if (p.D != 128) return MLSTM_E_UNSUPPORTED;
            return launch_fmt<DVC, 128>(p, in_dtype, out_dtype, st);
    }
    return MLSTM_E_ARG;
}

}  // namespace mlstm
