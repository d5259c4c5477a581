// Two-pass tensor-core form for head dimensions above 256, the shape of the reference's scan demo
// (mlstm_scan.py:375-394: S = 2048, D = 1024, where the D x D state of the recurrent form is larger
// than the S x S decay matrix, so the quadratic form is the one with the least arithmetic).
//
// It takes the place of the three contraction kernels of the reference's scan path
// (precompute_mlstm_triton_scan mlstm_scan.py:74-137, reduce_mlstm_triton :143-195, mlstm_triton_scan
// :200-278), which re-read K and Q once per 4 x 4 state patch.  Here every contraction is done once:
//
//   pass 1 (GATE)  W[r, c] = (q_r . k_c) * exp2(ec[c] + er[r])  for c <= r       [BH, S, S], causal part only
//                  one work item = 128 query rows x 256 key columns, contraction over the whole head
//                  dimension in 128-byte chunks; the gate factor, the causal mask and the partial row
//                  sums (the normaliser's b) are applied in the epilogue, W goes to a workspace that
//                  stays in L2 at the demo's size (33.5 MB written, read four times by pass 2)
//   pass 2 (APPLY) h[r, :] = (sum_c W[r, c] v_c) / n_r * silu(o_r)
//                  one work item = 128 query rows x 256 output columns, contraction over the causal
//                  extent of the row tile; n_r = max(|b_r|, exp(-m_r)) + 1e-6 from pass 1's row sums
//
// The parallel (matmul) path uses the same two passes above D = 256, forward and backward (run_group_bwd below:
// pass 1 for the normalised gated matrix and for its gradient, pass 2 for dQ and, with the matrix read
// MN-major as the A operand, for dK and dV).
//
// Both passes are the same persistent warp-specialised GEMM: warp 0 = TMA producer (ring of stages:
// a 128 x 128-byte A box and this CTA's share of B), warp 1 = MMA issuer (tcgen05.mma, N = 256, both
// operands from shared memory; fp32 inputs are read as tf32, 16-bit inputs as they are), warps 2-5 =
// epilogue (one TMEM lane = one row per thread; per-warp staging and TMA stores).  TMEM holds two
// 256-column accumulators, so the epilogue of one item overlaps the contraction of the next.  Work
// items come from a global counter, heaviest first, published to the roles through an eight-deep
// shared-memory ring.  Every wait is bounded (see ptx_sm100.cuh); a wait that runs out ends the
// kernel with a code in the status word.
//
// With fp32 operands a 128 x 256 tile needs 48 KB of operands for 512 cycles of MMA, and the measured
// rate of the copy engine into one SM (about 45 bytes per cycle here) makes both passes wait on loads.
// The PAIR form therefore runs on clusters of two CTAs (tcgen05.mma.cta_group::2, M = 256): an item is
// 256 query rows x 256 columns, each CTA loads its own 128 rows of A and HALF of B (32 KB per stage and
// CTA instead of 48 KB) and keeps its 128 rows of the accumulator in its own TMEM.  Signals that cross
// the pair as in mm_tc_pair.cu: loads of both CTAs count on the leader's "full" barrier, the leader's
// MMA thread commits to both CTAs' "empty" / "accumulator full" barriers, epilogue warps of both CTAs
// arrive on the leader's "accumulator drained" barrier, and work items travel from the leader's
// producer to the follower's through distributed shared memory.
#include <atomic>
#include <type_traits>

#include "mlstm_common.cuh"
#include "ptx_sm100.cuh"
#include "tc_host.cuh"

namespace mlstm {
namespace {

using namespace ptx;

constexpr int GATE = 0, APPLY = 1;
// pass 2: the tensor that comes in per-warp tiles beside the accumulator
constexpr int SIDE_NONE = 0;    // nothing
constexpr int SIDE_OGATE = 1;   // output gate o: the row is multiplied by silu(o)
constexpr int SIDE_DOT = 2;     // q resp. k: the row is dotted with it (the backward's R and dI vectors)
// Epilogue warps: pass 1 has eight (two per TMEM lane quarter, each taking every other 32-column chunk of the row:
// gating 256 elements per row with four warps took as long as the tile's contraction at D = 512), pass 2 four.
__host__ __device__ constexpr int nepi(int phase) { return phase == 0 ? 8 : 4; }
__host__ __device__ constexpr int nthreads_g(int phase) { return 64 + 32 * nepi(phase); }
constexpr int TN = 256;                       // columns of a work item
constexpr int A_BYTES = 128 * 128;            // 128 rows x 128 bytes
constexpr int B_BYTES = 256 * 128;            // pass 1: 256 key rows x 128 bytes; pass 2: TN columns x one chunk of rows
constexpr int OUT_WARP_BYTES = 2 * 2048;      // per epilogue warp: two staging buffers of 32 rows x 64 bytes
constexpr int ITEM_RING = 8;
constexpr int GATE_WARP_BYTES = 2 * 4096;     // pass 2, per epilogue warp: two tiles (32 rows x 128 bytes) of the output gate
template <bool PAIR, int PHASE>
struct GemmCfg {
    static constexpr int B_CTA = PAIR ? B_BYTES / 2 : B_BYTES;    // this CTA's share of B per stage
    static constexpr int STAGE = A_BYTES + B_CTA;
    static constexpr int NEPI = nepi(PHASE);
    static constexpr int IN_BYTES = PHASE == 1 ? NEPI * GATE_WARP_BYTES : 0;   // output-gate tiles of pass 2
    static constexpr int NSTAGE = PAIR ? (PHASE == 1 ? 5 : 6) : (PHASE == 1 ? 3 : 4);
    static constexpr int NBAR = 2 * NSTAGE + 4 + 2 * ITEM_RING + 2 * NEPI;
    static constexpr int SMEM = NSTAGE * STAGE + NEPI * OUT_WARP_BYTES + IN_BYTES + NBAR * 8 + 128;
    static_assert(SMEM <= 232448, "exceeds the shared memory of a CTA");
};
constexpr long long WAIT_LIMIT_G = 4000000000LL;   // cycles (about two seconds)
constexpr float MAX_ROW_EXP2_G = 60.0f;
constexpr int SLEEP_NS_G = 64;

struct GemmParams {
    int S, Spad, BH, D;
    int NT;        // 128-row tiles per slice
    int NP;        // pairs of row tiles per slice (PAIR form)
    int NKT;       // 256-column key tiles per slice
    int NVS;       // 256-column output slices
    int per_head;  // pass 1: work items per slice
    int items;     // work items of the launch
    // pass 1: gate vectors (see mlstm_common.cuh / gates.cu)
    const float* row_rel;
    const double* row_ref;
    const float* col_rel;
    const float* col_w;
    const double* col_ref;
    float er_add;
    const float* row_g; // [BH, Spad] added to every element of the row before the gate factor (backward), or nullptr
    float* bpart;       // [BH, 2 NKT, Spad] partial row sums, one per key tile and epilogue warp set, or nullptr
    // pass 2
    const float* m;     // [BH, S]; nullptr: rows are not normalised (backward)
    int side;           // what the [BH, S, D] tensor behind the fourth tensor map is: SIDE_NONE, SIDE_OGATE, SIDE_DOT
    float* b_out;       // [BH, S] row sums (optional)
    float* dot_out;     // SIDE_DOT: [NVS][BH, Spad] row dots, one partial per 256-column output slice
    long long dot_stride;
    int* status;
    int* counter;       // work-item counter of this launch (zeroed by the launcher)
};

__device__ __forceinline__ uint32_t to_tf32_rn(float x) {
    uint32_t y;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(y) : "f"(x));
    return y;
}

// at most `N` of this thread's bulk groups are still reading their shared-memory source
template <int N>
__device__ __forceinline__ void bulk_wait_read() {
    asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}

// TRANS (pass 2 only): the contraction runs over the ROWS of the S x S matrix, out[c, :] = sum_r M[r, c] Z[r, :] for
// r >= c (the backward's dK and dV): the A operand is the matrix read MN-major, in the same boxes as B.
// OUT_IN (pass 2 only): the output has the inputs' element type (gradients) instead of fp32 (h).
template <int PHASE, int ABFMT, bool PAIR, bool TRANS = false, bool OUT_IN = false>
__global__ void __launch_bounds__(nthreads_g(PHASE), 1)
mlstm_scan_gemm(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                const __grid_constant__ CUtensorMap tmO, const __grid_constant__ CUtensorMap tmG, const GemmParams p) {
    using G = GemmCfg<PAIR, PHASE>;
    constexpr int NEPI = G::NEPI;
    constexpr int NSTAGE = G::NSTAGE;
    constexpr int STAGE_BYTES_G = G::STAGE;
    constexpr int NBAR_G = G::NBAR;
    constexpr bool TF32 = ABFMT == 2;
    constexpr int ES = TF32 ? 4 : 2;
    constexpr int KC = 128 / ES;                 // contraction elements per stage (one 128-byte row)
    constexpr int KSTEP = 32 / ES;               // contraction elements per MMA
    using InT = typename std::conditional<ABFMT == 2, float,
                                          typename std::conditional<ABFMT == 1, __nv_bfloat16, __half>::type>::type;
    static_assert(PHASE == APPLY || (!TRANS && !OUT_IN), "pass 1 has one form");
    // pass 1 writes W in the input type, pass 2 writes h in fp32 or gradients in the input type
    constexpr int OUT_ES = (PHASE == GATE || OUT_IN) ? ES : 4;
    constexpr int NSUB = OUT_ES == 4 ? 2 : 1;    // TMA stores of 64 bytes per row for a 32-column chunk
    // pass 2: B boxes are KC rows x 128 bytes, one per 128-byte column group of the item's 256 columns
    constexpr int B2_BOX = KC * 128;
    constexpr int B2_GROUPS = TN * ES / 128;
    constexpr int AT_GROUPS = TILE * ES / 128;   // TRANS: 128-byte column groups of a row tile's 128 matrix columns

    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t* smem = smem_raw;
    uint8_t* sOut = smem + NSTAGE * STAGE_BYTES_G;
    uint8_t* sIn = sOut + NEPI * OUT_WARP_BYTES;      // pass 2: output-gate tiles (1024-byte aligned: stages and staging are)
    uint64_t* bars = reinterpret_cast<uint64_t*>(sIn + G::IN_BYTES);
    uint64_t* bar_full = bars;
    uint64_t* bar_empty = bars + NSTAGE;
    uint64_t* bar_accfull = bars + 2 * NSTAGE;        // [2]
    uint64_t* bar_accempty = bar_accfull + 2;         // [2]
    uint64_t* bar_item = bar_accempty + 2;            // [ITEM_RING] work item published inside the CTA
    uint64_t* bar_item_in = bar_item + ITEM_RING;     // [ITEM_RING] PAIR, follower: work item arrived from the leader
    uint64_t* bar_gate = bar_item_in + ITEM_RING;     // [NEPI][2] pass 2: output-gate tile loaded (one pair per epilogue warp)
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + NBAR_G);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    volatile int* item_ids = reinterpret_cast<volatile int*>(tmem_slot + 2);                 // [ITEM_RING]
    volatile int* item_in = reinterpret_cast<volatile int*>(tmem_slot + 2 + ITEM_RING);      // [ITEM_RING]

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const bool misaligned = (smem_u32(smem) & 1023u) != 0;   // the swizzled tiles need a 1024-byte aligned base
    const uint32_t rank = PAIR ? cluster_ctarank() : 0u;      // 0 = leader
    auto at_leader = [&](const void* local) { return mapa_u32(smem_u32(local), 0u); };
    auto at_peer = [&](const void* local) { return mapa_u32(smem_u32(local), rank ^ 1u); };

    // qt: this CTA's 128-row tile (PAIR: tile 2 * pair + rank, which may lie past the end of an odd-length slice:
    // such a half loads zeros and only keeps the protocol going); ct: key tile (pass 1) or output slice (pass 2)
    struct Item {
        int bh, qt, ct, nchunks;
    };
    auto decode = [&](int id) {
        Item it;
        if (PHASE == GATE) {
            it.bh = id / p.per_head;
            int idx = id - it.bh * p.per_head;
            int g = 0;   // row tile (PAIR: pair of row tiles) g has ntiles(g) key tiles on or below its diagonal
            while (idx >= (PAIR ? g + 1 : g / 2 + 1)) {
                idx -= PAIR ? g + 1 : g / 2 + 1;
                g++;
            }
            it.qt = PAIR ? 2 * g + static_cast<int>(rank) : g;
            it.ct = idx;
            it.nchunks = p.D / KC;
        } else {
            const int per_w = p.BH * p.NVS;
            const int w = id / per_w;
            const int rem = id - w * per_w;
            const int g = TRANS ? w : (PAIR ? p.NP : p.NT) - 1 - w;   // longest contractions first
            it.qt = PAIR ? 2 * g + static_cast<int>(rank) : g;
            it.bh = rem / p.NVS;
            it.ct = rem - it.bh * p.NVS;
            // the causal extent of the (pair's lower) row tile; the gated matrix holds zeros right of a tile's diagonal.
            // TRANS: the matrix rows from the (pair's upper) tile's first one to the end.
            if (TRANS) it.nchunks = (p.Spad - (PAIR ? 2 * g : g) * TILE) / KC;
            else it.nchunks = (PAIR ? min((2 * g + 2) * TILE, p.Spad) : (g + 1) * TILE) / KC;
        }
        return it;
    };

    if (threadIdx.x == 0) {
        for (int s = 0; s < NSTAGE; s++) {
            mbar_init(&bar_full[s], 1);
            mbar_init(&bar_empty[s], 1);
        }
        for (int k = 0; k < 2; k++) {
            mbar_init(&bar_accfull[k], 1);
            mbar_init(&bar_accempty[k], PAIR ? 2 * NEPI : NEPI);
        }
        for (int k = 0; k < ITEM_RING; k++) {
            mbar_init(&bar_item[k], 1);
            mbar_init(&bar_item_in[k], 1);
        }
        for (int k = 0; k < 2 * NEPI; k++) mbar_init(&bar_gate[k], 1);
        *abort_flag = misaligned ? 1 : 0;
        fence_mbar_init();
    }
    if (warp == 1) {
        if constexpr (PAIR) {
            tmem_alloc_pair(tmem_slot, 512);
            tmem_relinquish_pair();
        } else {
            tmem_alloc(tmem_slot, 512);
            tmem_relinquish();
        }
    }
    tc_fence_before();
    __syncthreads();
    if constexpr (PAIR) cluster_sync_all();   // the peer's barriers are initialised before anything signals them
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    // Everything above (barriers, TMEM, tensor-map fetches come later) touched no global memory: it may run under the tail
    // of the kernel before this one in the stream (the gate pass, or pass 1).  From here on that kernel's results are needed.
    grid_dep_wait();
    grid_dep_launch();

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer
        if (lane == 0 && !misaligned) {
            prefetch_tmap(&tmA);
            prefetch_tmap(&tmB);
            int seq = 0;   // stages filled so far
            bool ok = true;
            for (int n = 0; ok; n++) {
                int id;
                if (rank == 0) {
                    id = atomicAdd(p.counter, 1);
                    if (id >= p.items) id = -1;
                    if constexpr (PAIR) {   // to the follower's producer: cluster-scope release, once per item
                        st_cluster_u32(at_peer(const_cast<int*>(&item_in[n % ITEM_RING])), static_cast<uint32_t>(id));
                        mbar_arrive_cluster(at_peer(&bar_item_in[n % ITEM_RING]));
                    }
                } else {
                    ok = mbar_wait_cluster<SLEEP_NS_G>(&bar_item_in[n % ITEM_RING], (n / ITEM_RING) & 1, abort_flag, WAIT_LIMIT_G);
                    id = ok ? item_in[n % ITEM_RING] : -1;
                }
                item_ids[n % ITEM_RING] = id;
                mbar_arrive(&bar_item[n % ITEM_RING]);   // release: the id is visible to whoever passes the wait
                if (id < 0) break;
                const Item it = decode(id);
                for (int c = 0; c < it.nchunks && ok; c++, seq++) {
                    const int s = seq % NSTAGE;
                    if (seq >= NSTAGE) {
                        ok = mbar_wait<SLEEP_NS_G>(&bar_empty[s], ((seq / NSTAGE) & 1) ^ 1, abort_flag, WAIT_LIMIT_G);
                        if (!ok) break;
                    }
                    uint8_t* sa = smem + s * STAGE_BYTES_G;
                    uint8_t* sb = sa + A_BYTES;
                    // A: rows of this CTA's query tile, one 128-byte chunk of the contraction (pass 1: of the head
                    // dimension of Q; pass 2: of the key positions of W).  B, pass 1: key rows of the same chunk (PAIR:
                    // this CTA's 128 of the 256); pass 2: KC value rows x the item's columns (PAIR: this CTA's half of
                    // them), all 128-byte column groups with ONE copy (a copy per group made the pass wait on the copy
                    // engine: nine copies per stage ran at 2900 cycles per stage)
                    // TRANS: chunk c is KC matrix rows from the item's first one; A = this CTA's 128 matrix columns of them
                    // (all their 128-byte groups with one copy, like B), B = the same rows of Z
                    const int k0 = TRANS ? (PAIR ? it.qt - static_cast<int>(rank) : it.qt) * TILE + c * KC : c * KC;
                    if constexpr (PAIR) {
                        if (rank == 0) mbar_expect_tx(&bar_full[s], 2 * STAGE_BYTES_G);   // the loads of both CTAs
                        const uint32_t lead_full = at_leader(&bar_full[s]);
                        if (TRANS) tma_load_4d_pair(sa, &tmA, lead_full, 0, k0, it.qt * AT_GROUPS, it.bh);
                        else tma_load_3d_pair(sa, &tmA, lead_full, k0, it.qt * TILE, it.bh);
                        if (PHASE == GATE)
                            tma_load_3d_pair(sb, &tmB, lead_full, k0, it.ct * TN + static_cast<int>(rank) * (TN / 2), it.bh);
                        else
                            tma_load_4d_pair(sb, &tmB, lead_full, 0, k0,
                                             it.ct * B2_GROUPS + static_cast<int>(rank) * (B2_GROUPS / 2), it.bh);
                    } else {
                        mbar_expect_tx(&bar_full[s], STAGE_BYTES_G);
                        if (TRANS) tma_load_4d(sa, &tmA, &bar_full[s], 0, k0, it.qt * AT_GROUPS, it.bh);
                        else tma_load_3d(sa, &tmA, &bar_full[s], k0, it.qt * TILE, it.bh);
                        if (PHASE == GATE) tma_load_3d(sb, &tmB, &bar_full[s], k0, it.ct * TN, it.bh);
                        else tma_load_4d(sb, &tmB, &bar_full[s], 0, k0, it.ct * B2_GROUPS, it.bh);
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer (PAIR: the leader's, for both CTAs)
        if (rank == 0) {
        // the whole warp runs the loop, one elected lane issues (tcgen05.mma wants warp-uniform operands)
        const bool issuer = elect_one();
        auto uni = [](int x) { return __shfl_sync(0xffffffffu, x, 0); };
        auto wait_u = [&](uint64_t* bar, uint32_t parity) { return mbar_wait_warp(bar, parity, abort_flag, WAIT_LIMIT_G); };
        constexpr uint32_t idesc = make_idesc(ABFMT, PAIR ? 256 : 128, TN, TRANS ? 1 : 0, PHASE == GATE ? 0 : 1);
        const uint32_t smem_u = static_cast<uint32_t>(uni(static_cast<int>(smem_u32(smem))));
        const uint32_t tmem_u = static_cast<uint32_t>(uni(static_cast<int>(tmem_base)));
        const uint32_t bars_u = smem_u + NSTAGE * STAGE_BYTES_G + NEPI * OUT_WARP_BYTES + G::IN_BYTES;        // this CTA's barriers ...
        const uint32_t bars_peer_u = PAIR ? static_cast<uint32_t>(uni(static_cast<int>(at_peer(bars)))) : 0u;   // ... and the peer's
        auto commit = [&](const uint64_t* bar) {   // one arrival (PAIR: in either CTA) once the MMAs issued so far are done
            if constexpr (PAIR) {
                const uint32_t off = static_cast<uint32_t>(bar - bars) * 8u;
                tc_commit_pair(bars_u + off);
                tc_commit_pair(bars_peer_u + off);
            } else {
                tc_commit(const_cast<uint64_t*>(bar));
            }
        };
        const uint64_t adesc0 = !TRANS ? smem_desc_sw128(smem_u, 16, 1024)              // K-major, 128-byte rows
                                : (TF32 ? smem_desc_sw128(smem_u, B2_BOX, 512, 1)        // MN-major like B of pass 2
                                        : smem_desc_sw128(smem_u, B2_BOX, 1024, 2));
        constexpr int A_KSTEP_BYTES = TRANS ? KSTEP * 128 : 32;          // advance of A per MMA
        const uint64_t bdesc0 = PHASE == GATE ? smem_desc_sw128(smem_u + A_BYTES, 16, 1024)           // K-major, 256 rows
                                : (TF32 ? smem_desc_sw128(smem_u + A_BYTES, B2_BOX, 512, 1)          // MN-major, 32-bit
                                        : smem_desc_sw128(smem_u + A_BYTES, B2_BOX, 1024, 2));        // MN-major, 16-bit
        constexpr int B_KSTEP_BYTES = PHASE == GATE ? 32 : KSTEP * 128;   // advance of B per MMA
        int seq = 0;
        bool ok = __all_sync(0xffffffffu, *abort_flag ? 0 : 1) != 0;
        for (int n = 0; ok; n++) {
            ok = wait_u(&bar_item[n % ITEM_RING], (n / ITEM_RING) & 1);
            if (!ok) break;
            const int id = uni(item_ids[n % ITEM_RING]);
            if (id < 0) break;
            const Item it = decode(id);
            const int buf = n & 1;
            if (n >= 2) {   // the epilogue of the item before last has drained this accumulator
                ok = wait_u(&bar_accempty[buf], ((n >> 1) & 1) ^ 1);
                if (!ok) break;
                tc_fence_after();
            }
            const uint32_t acc = tmem_u + buf * TN;
            for (int c = 0; c < it.nchunks && ok; c++, seq++) {
                const int s = seq % NSTAGE;
                ok = wait_u(&bar_full[s], (seq / NSTAGE) & 1);
                if (!ok) break;
                if (issuer) {
                    const uint64_t ad = smem_desc_advance(adesc0, s * STAGE_BYTES_G);
                    const uint64_t bd = smem_desc_advance(bdesc0, s * STAGE_BYTES_G);
#pragma unroll
                    for (int kk = 0; kk < KC / KSTEP; kk++) {
                        if constexpr (PAIR)
                            mma_ss_pair_fmt<TF32>(acc, smem_desc_advance(ad, kk * A_KSTEP_BYTES),
                                                  smem_desc_advance(bd, kk * B_KSTEP_BYTES), idesc, (c > 0 || kk > 0) ? 1u : 0u);
                        else
                            mma_ss<TF32>(acc, smem_desc_advance(ad, kk * A_KSTEP_BYTES), smem_desc_advance(bd, kk * B_KSTEP_BYTES),
                                         idesc, (c > 0 || kk > 0) ? 1u : 0u);
                    }
                    commit(&bar_empty[s]);
                    if (c == it.nchunks - 1) commit(&bar_accfull[buf]);
                }
                __syncwarp();
            }
        }
        }   // rank == 0
    } else {
        // ------------------------------------------------------------ epilogue warps
        const int r = (warp & 3) * 32 + lane;          // TMEM lane == row inside the tile (lane quarter = warp % 4)
        const uint32_t lane_bits = static_cast<uint32_t>((warp & 3) * 32) << 16;
        // with eight epilogue warps two share a lane quarter: warp set e takes the chunks ch = e, e + 2, ...
        constexpr int NSET = NEPI / 4;
        const int eset = (warp - 2) >> 2;
        uint8_t* stage = sOut + (warp - 2) * OUT_WARP_BYTES;
        if (lane == 0) prefetch_tmap(&tmO);
        // Pass 2: the output gate o of this warp's 32 rows comes in tiles of 32 rows x 128 bytes through the copy
        // engine, two tiles ahead of their use (per-thread loads of a row each, 32 lines per instruction, were what
        // the whole pass waited for: 75 of its 100 microseconds at the reference demo's size).
        [[maybe_unused]] uint8_t* gate_buf = sIn + (warp - 2) * GATE_WARP_BYTES;
        [[maybe_unused]] uint64_t* gate_bar = bar_gate + (warp - 2) * 2;
        [[maybe_unused]] int ngate = 0;   // gate tiles consumed by this warp: buffer and barrier phase follow it
        constexpr int GATE_COLS = 128 / ES;               // columns of o per tile
        constexpr int GATE_TILES = TN / GATE_COLS;        // tiles per item and warp
        constexpr int GATE_TILE_BYTES = 32 * 128;
        [[maybe_unused]] const bool gated = PHASE == APPLY && p.side != SIDE_NONE;   // a side tensor comes in tiles
        [[maybe_unused]] const bool side_dot = PHASE == APPLY && p.side == SIDE_DOT;
        if (PHASE == APPLY && lane == 0) prefetch_tmap(&tmG);
        int nstore = 0;   // stores issued by this warp: alternates its two staging buffers
        bool ok = __all_sync(0xffffffffu, *abort_flag ? 0 : 1) != 0;
        // 32 rows x 64 bytes of `vals` (16 fp32 or 32 16-bit values per row, already converted) to global memory
        auto store64 = [&](const uint4 (&v)[4], int x, int y, int z) {
            uint8_t* buf = stage + (nstore & 1) * 2048;
            if (lane == 0) bulk_wait_read<1>();    // the store before last has read this buffer
            __syncwarp();
            uint4* srow = reinterpret_cast<uint4*>(buf + lane * 64);
            const int sw = (lane >> 1) & 3;        // 64-byte swizzle of the store's tensor map: no bank conflicts
#pragma unroll
            for (int j4 = 0; j4 < 4; j4++) srow[j4 ^ sw] = v[j4];
            fence_async_smem();
            __syncwarp();
            if (lane == 0) {
                tma_store_3d(&tmO, buf, x, y, z);
                bulk_commit();
            }
            nstore++;
        };
        for (int n = 0; ok; n++) {
            ok = mbar_wait_warp<SLEEP_NS_G>(&bar_item[n % ITEM_RING], (n / ITEM_RING) & 1, abort_flag, WAIT_LIMIT_G);
            if (!ok) break;
            const int id = __shfl_sync(0xffffffffu, item_ids[n % ITEM_RING], 0);
            if (id < 0) break;
            const Item it = decode(id);
            const int buf = n & 1;
            const int grow = it.qt * TILE + r;
            const bool active = it.qt < p.NT;      // PAIR: the second half of an odd last pair has no rows
            const bool row_ok = grow < p.S;
            auto load_gate_tile = [&](int tile, int seq) {   // lane 0: tile `tile` of this item into buffer seq & 1
                mbar_expect_tx(&gate_bar[seq & 1], GATE_TILE_BYTES);
                tma_load_3d(gate_buf + (seq & 1) * GATE_TILE_BYTES, &tmG, &gate_bar[seq & 1], it.ct * TN + tile * GATE_COLS,
                            it.qt * TILE + (warp & 3) * 32, it.bh);
            };
            if (gated && active && lane == 0) {
                load_gate_tile(0, ngate);
                load_gate_tile(1, ngate + 1);
            }
            const size_t vec_base = static_cast<size_t>(it.bh) * p.Spad;
            const size_t ref_base = static_cast<size_t>(it.bh) * (p.Spad / REF_BLOCK);
            // row terms, requested before the accumulator wait
            double er_d = 0.0;
            float inv_n = 1.0f;
            [[maybe_unused]] float g_row = 0.0f, dot = 0.0f;
            if (!active) {
                // nothing to read: the accumulator holds zeros and nothing is stored
            } else if (PHASE == GATE) {
                er_d = static_cast<double>(p.row_rel[vec_base + grow]) + p.row_ref[ref_base + grow / REF_BLOCK] +
                       static_cast<double>(p.er_add);
                if (p.row_g) g_row = p.row_g[vec_base + grow];
            } else if (p.m) {
                float bsum = 0.0f;
                constexpr int PARTS_PER_TILE = nepi(GATE) / 4;   // pass 1 wrote one partial per key tile and warp set
                for (int kt = 0; kt < (it.qt / 2 + 1) * PARTS_PER_TILE; kt++)
                    bsum += p.bpart[(static_cast<size_t>(it.bh) * p.NKT * PARTS_PER_TILE + kt) * p.Spad + grow];
                const float mrow = row_ok ? p.m[static_cast<size_t>(it.bh) * p.S + grow] : 0.0f;
                inv_n = 1.0f / (fmaxf(fabsf(bsum), __expf(-mrow)) + 1e-6f);
                if (p.b_out && it.ct == 0 && row_ok) p.b_out[static_cast<size_t>(it.bh) * p.S + grow] = bsum;
            }
            ok = mbar_wait_warp<SLEEP_NS_G>(&bar_accfull[buf], (n >> 1) & 1, abort_flag, WAIT_LIMIT_G);
            if (!ok) break;
            tc_fence_after();
            const uint32_t acc = tmem_base + buf * TN + lane_bits;
            float rowsum = 0.0f;
            // pass 1: chunks right of the row tile's diagonal tile are never read by pass 2: not computed, not stored
            const int nch = !active ? 0 : (PHASE == GATE ? min(TN / 32, ((it.qt + 1) * TILE - it.ct * TN) / 32) : TN / 32);
            auto release_acc = [&]() {   // this warp's share of the accumulator is in registers (or not needed)
                tc_fence_before();
                __syncwarp();
                if (lane == 0) {
                    if constexpr (PAIR) mbar_arrive_remote(at_leader(&bar_accempty[buf]));
                    else mbar_arrive(&bar_accempty[buf]);
                }
            };
            if (nch <= eset) release_acc();     // (nch is a multiple of four: every warp set has chunks, or none has)
#pragma unroll 1
            for (int ch = eset; ch < nch; ch += NSET) {
                const int c0 = it.ct * TN + ch * 32;           // first column of the chunk (pass 1: key position)
                float cv[32];
                bool diag = false;
                float er = 0.0f;
                if (PHASE == GATE) {
                    diag = (c0 / TILE) == it.qt;
                    const float4* p4 = reinterpret_cast<const float4*>((diag ? p.col_rel : p.col_w) + vec_base + c0);
#pragma unroll
                    for (int q4 = 0; q4 < 8; q4++) {
                        const float4 e4 = __ldg(p4 + q4);
                        cv[q4 * 4 + 0] = e4.x; cv[q4 * 4 + 1] = e4.y; cv[q4 * 4 + 2] = e4.z; cv[q4 * 4 + 3] = e4.w;
                    }
                    er = static_cast<float>(er_d + p.col_ref[ref_base + c0 / REF_BLOCK]);
                } else if (gated) {
                    // 32 columns of this row from the warp's gate tile (128-byte swizzle: the 16-byte piece j of row
                    // r sits at piece j ^ (r & 7)); a tile holds GATE_COLS columns, i.e. one or two chunks
                    constexpr int VEC = 16 / ES;
                    constexpr int CH_PER_TILE = GATE_COLS / 32;
                    const int tile = ch / CH_PER_TILE, sub = ch % CH_PER_TILE;
                    const int seq = ngate + tile;
                    if (sub == 0) {
                        ok = mbar_wait_warp<SLEEP_NS_G>(&gate_bar[seq & 1], (seq >> 1) & 1, abort_flag, WAIT_LIMIT_G);
                        if (!ok) break;
                    }
                    const uint8_t* grow_smem = gate_buf + (seq & 1) * GATE_TILE_BYTES + lane * 128;
#pragma unroll
                    for (int jv = 0; jv < 32 / VEC; jv++) {
                        const int piece = sub * (32 / VEC) + jv;
                        const uint4 raw = *reinterpret_cast<const uint4*>(grow_smem + ((piece ^ (lane & 7)) << 4));
                        const InT* ev = reinterpret_cast<const InT*>(&raw);
#pragma unroll
                        for (int j = 0; j < VEC; j++) cv[jv * VEC + j] = side_dot ? to_f32<InT>(ev[j]) : silu_f(to_f32<InT>(ev[j]));
                    }
                    if (sub == CH_PER_TILE - 1) {   // the tile is in registers: fetch the tile after next into its buffer
                        __syncwarp();
                        if (lane == 0 && tile + 2 < GATE_TILES) load_gate_tile(tile + 2, seq + 2);
                    }
                } else {
#pragma unroll
                    for (int j = 0; j < 32; j++) cv[j] = 1.0f;
                }
                uint32_t tv[32];
                tmem_ld32(acc + ch * 32, tv);
                tc_wait_ld();
                if (ch + NSET >= nch) release_acc();   // this warp's last chunk: the item after next may overwrite the accumulator
                if (PHASE == GATE) {
                    if (diag) {
                        const int rel0 = c0 - it.qt * TILE;    // column index inside the diagonal tile
#pragma unroll
                        for (int j = 0; j < 32; j++) {
                            float wj = (__uint_as_float(tv[j]) + g_row) * fast_exp2(cv[j] + er);
                            if (rel0 + j > r) wj = 0.0f;
                            rowsum += wj;
                            cv[j] = wj;
                        }
                    } else {
                        // off the diagonal tile exp2(ec + er) = exp2(ec) exp2(er) with both factors bounded; a
                        // block of pure padding has no reference of its own, hence the clamp (its factors are 0)
                        const float u = fast_exp2(fminf(er, MAX_ROW_EXP2_G));
                        const float gu = g_row * u;
#pragma unroll
                        for (int j = 0; j < 32; j++) {
                            const float wj = fmaf(__uint_as_float(tv[j]), u, gu) * cv[j];
                            rowsum += wj;
                            cv[j] = wj;
                        }
                    }
                } else if (side_dot) {
#pragma unroll
                    for (int j = 0; j < 32; j++) {
                        const float x = __uint_as_float(tv[j]);
                        dot = fmaf(x, cv[j], dot);
                        cv[j] = x;
                    }
                } else {
#pragma unroll
                    for (int j = 0; j < 32; j++) cv[j] *= __uint_as_float(tv[j]) * inv_n;
                }
                const int y = it.qt * TILE + (warp & 3) * 32;
                if constexpr (OUT_ES == 4) {
#pragma unroll
                    for (int sub = 0; sub < NSUB; sub++) {
                        uint4 v[4];
#pragma unroll
                        for (int j4 = 0; j4 < 4; j4++) {
                            const float* s4 = &cv[sub * 16 + j4 * 4];
                            if (PHASE == GATE)
                                v[j4] = make_uint4(to_tf32_rn(s4[0]), to_tf32_rn(s4[1]), to_tf32_rn(s4[2]), to_tf32_rn(s4[3]));
                            else
                                v[j4] = make_uint4(__float_as_uint(s4[0]), __float_as_uint(s4[1]), __float_as_uint(s4[2]),
                                                   __float_as_uint(s4[3]));
                        }
                        store64(v, c0 + sub * 16, y, it.bh);
                    }
                } else {
                    uint4 v[4];
#pragma unroll
                    for (int j4 = 0; j4 < 4; j4++) {
                        uint32_t o32[4];
#pragma unroll
                        for (int j = 0; j < 4; j++) {
                            if constexpr (ABFMT == 1) {
                                __nv_bfloat162 v2 = __floats2bfloat162_rn(cv[j4 * 8 + 2 * j], cv[j4 * 8 + 2 * j + 1]);
                                o32[j] = *reinterpret_cast<uint32_t*>(&v2);
                            } else {
                                __half2 v2 = __floats2half2_rn(cv[j4 * 8 + 2 * j], cv[j4 * 8 + 2 * j + 1]);
                                o32[j] = *reinterpret_cast<uint32_t*>(&v2);
                            }
                        }
                        v[j4] = make_uint4(o32[0], o32[1], o32[2], o32[3]);
                    }
                    store64(v, c0, y, it.bh);
                }
            }
            if (!ok) break;
            if (gated && active) ngate += GATE_TILES;
            if (side_dot && active && p.dot_out)
                p.dot_out[it.ct * p.dot_stride + static_cast<long long>(vec_base) + grow] = row_ok ? dot : 0.0f;
            if (PHASE == GATE && active) {
                // one partial per key tile and warp set
                if (p.bpart) p.bpart[(static_cast<size_t>(it.bh) * p.NKT * NSET + it.ct * NSET + eset) * p.Spad + grow] = rowsum;
                if constexpr (PAIR) {
                    // Pass 2 contracts a pair of row tiles over the causal extent of the lower one.  For the upper tile
                    // that includes the 128 columns right of its diagonal tile, which nothing computes: they must read
                    // as zeros (the workspace may hold anything).
                    if (rank == 0 && it.ct * TN + nch * 32 < min((it.qt + 2) * TILE, p.Spad) && it.ct == it.qt / 2) {
                        uint4 z[4];
#pragma unroll
                        for (int j4 = 0; j4 < 4; j4++) z[j4] = make_uint4(0u, 0u, 0u, 0u);
                        const int y = it.qt * TILE + (warp & 3) * 32;
                        for (int ch = nch + eset; ch < TN / 32; ch += NSET) {
                            const int c0 = it.ct * TN + ch * 32;
#pragma unroll
                            for (int sub = 0; sub < NSUB; sub++) store64(z, c0 + sub * (64 / OUT_ES), y, it.bh);
                        }
                    }
                }
            }
        }
        if (lane == 0) bulk_wait_all();   // the last stores have left shared memory before the CTA goes away
        tc_fence_before();
    }

    __syncthreads();
    if (*abort_flag) {
        if (threadIdx.x == 0) atomicExch(p.status, misaligned ? 2000 : 5000 + PHASE);
        // give copies and MMAs that are still in flight time to land before the CTA's memory goes away
        for (int k = 0; k < 64; k++) __nanosleep(16000);
        __syncthreads();
    }
    if constexpr (PAIR) cluster_sync_all();   // neither CTA releases shared memory or TMEM the other may still touch
    if (warp == 1) {
        tc_fence_after();
        if constexpr (PAIR) tmem_dealloc_pair(tmem_base, 512);
        else tmem_dealloc(tmem_base, 512);
    }
}

template <int PHASE, int ABFMT, bool PAIR, bool TRANS = false, bool OUT_IN = false>
int launch_gemm(const CUtensorMap& ma, const CUtensorMap& mb, const CUtensorMap& mo, const CUtensorMap& mg, const GemmParams& p,
                bool zero_counter, cudaStream_t st) {
    auto kern = mlstm_scan_gemm<PHASE, ABFMT, PAIR, TRANS, OUT_IN>;
    constexpr int smem = GemmCfg<PAIR, PHASE>::SMEM;
    cudaError_t ce;
    {
        static std::atomic<bool> opted[64];
        int dev = 0;
        if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return MLSTM_E_CUDA;
        if (!opted[dev].load(std::memory_order_acquire)) {
            ce = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
            if (ce != cudaSuccess) {
                cudaGetLastError();
                return note_cuda_error(ce, "cudaFuncSetAttribute(MaxDynamicSharedMemorySize)");
            }
            opted[dev].store(true, std::memory_order_release);
        }
    }
    const int sms = tc_sm_count();
    if (sms <= 0) return MLSTM_E_CUDA;
    if (zero_counter) {
        ce = cudaMemsetAsync(p.counter, 0, sizeof(int), st);
        if (ce != cudaSuccess) return note_cuda_error(ce, "cudaMemsetAsync(item counter)");
    }
    // persistent: one CTA (PAIR: one CTA of a cluster of two) per SM
    const int units = PAIR ? sms / 2 : sms;
    const int n = p.items < units ? p.items : units;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(static_cast<unsigned>(PAIR ? 2 * n : n), 1, 1);
    cfg.blockDim = dim3(nthreads_g(PHASE), 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = PAIR ? 2 : 1;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;   // see grid_dep_wait() in the kernel
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 2;
    ce = cudaLaunchKernelEx(&cfg, kern, ma, mb, mo, mg, p);
    if (ce != cudaSuccess) {
        cudaGetLastError();
        return note_cuda_error(ce, "launch of mlstm_scan_gemm");
    }
    return MLSTM_OK;
}

// The pair form needs at least two row tiles per slice and two SMs; a single tile runs on one CTA.
inline bool use_pairs(int Spad) { return Spad > TILE && tc_sm_count() >= 2; }

template <int ABFMT, bool PAIR>
int run_group(const void* q, const void* k, const void* v, const void* o, float* h, void* W, const ScanGemmArgs& a, int bh0,
              int nbh, int dtype, cudaStream_t st) {
    const bool zero_counters = bh0 > 0;   // the gate pass cleared both counters with the status word for the first group
    const size_t es = dtype == MLSTM_DT_F32 ? 4 : 2;
    const size_t slice = static_cast<size_t>(a.S) * a.D;
    const uint8_t* qg = static_cast<const uint8_t*>(q) + bh0 * slice * es;
    const uint8_t* kg = static_cast<const uint8_t*>(k) + bh0 * slice * es;
    const uint8_t* vg = static_cast<const uint8_t*>(v) + bh0 * slice * es;
    const uint8_t* og = o ? static_cast<const uint8_t*>(o) + bh0 * slice * es : nullptr;
    float* hg = h + bh0 * slice;
    GemmParams p{};
    p.S = a.S; p.Spad = a.Spad; p.BH = nbh; p.D = a.D;
    p.NT = a.Spad / TILE;
    p.NP = (p.NT + 1) / 2;
    p.NKT = (a.Spad + TN - 1) / TN;
    p.NVS = a.D / TN;
    p.per_head = 0;
    if (PAIR) for (int g = 0; g < p.NP; g++) p.per_head += g + 1;
    else for (int qt = 0; qt < p.NT; qt++) p.per_head += qt / 2 + 1;
    const size_t vec0 = static_cast<size_t>(bh0) * a.Spad, ref0 = static_cast<size_t>(bh0) * (a.Spad / REF_BLOCK);
    p.row_rel = a.gAn + vec0; p.row_ref = a.An_ref + ref0;
    p.col_rel = a.ga + vec0; p.col_w = a.gaw + vec0; p.col_ref = a.a_ref + ref0;
    p.er_add = -0.5f * log2f(static_cast<float>(a.D));
    p.bpart = a.bpart;   // per group: reused
    p.m = a.m + static_cast<size_t>(bh0) * a.S;
    p.side = og ? SIDE_OGATE : SIDE_NONE;
    p.b_out = a.b ? a.b + static_cast<size_t>(bh0) * a.S : nullptr;
    p.status = a.status;
    int rc;
    CUtensorMap ma, mb, mo;
    // ---- pass 1: W = gate(Q K^T)
    if ((rc = tc_make_map(&ma, qg, nbh, a.S, a.D, dtype, false, 128)) != MLSTM_OK) return rc;
    if ((rc = tc_make_map(&mb, kg, nbh, a.S, a.D, dtype, false, PAIR ? TN / 2 : TN)) != MLSTM_OK) return rc;
    if ((rc = tc_make_map_out(&mo, W, nbh, a.Spad, a.Spad, dtype, 32)) != MLSTM_OK) return rc;
    p.items = p.per_head * nbh;
    p.counter = a.counters;
    if ((rc = launch_gemm<GATE, ABFMT, PAIR>(ma, mb, mo, mo, p, zero_counters, st)) != MLSTM_OK) return rc;
    // ---- pass 2: h = (W V) / n * silu(o)
    constexpr int KC = ABFMT == 2 ? 32 : 64;
    constexpr int GROUPS = TN * (ABFMT == 2 ? 4 : 2) / 128;   // 128-byte column groups of an item's 256 columns
    if ((rc = tc_make_map(&ma, W, nbh, a.Spad, a.Spad, dtype, false, 128)) != MLSTM_OK) return rc;
    if ((rc = tc_make_map_groups(&mb, vg, nbh, a.S, a.D, dtype, ABFMT == 2, KC, PAIR ? GROUPS / 2 : GROUPS)) != MLSTM_OK) return rc;
    if ((rc = tc_make_map_out(&mo, hg, nbh, a.S, a.D, MLSTM_DT_F32, 32)) != MLSTM_OK) return rc;
    CUtensorMap mg = mo;   // output gate: tiles of 32 rows x 128 bytes, one per epilogue warp and step
    if (og && (rc = tc_make_map(&mg, og, nbh, a.S, a.D, dtype, false, 32)) != MLSTM_OK) return rc;
    p.items = (PAIR ? p.NP : p.NT) * nbh * p.NVS;
    p.counter = a.counters + 1;
    return launch_gemm<APPLY, ABFMT, PAIR>(ma, mb, mo, mg, p, zero_counters, st);
}

template <int ABFMT>
int run_group_any(const void* q, const void* k, const void* v, const void* o, float* h, void* W, const ScanGemmArgs& a, int bh0,
                  int nbh, int dtype, cudaStream_t st) {
    if (use_pairs(a.Spad)) return run_group<ABFMT, true>(q, k, v, o, h, W, a, bh0, nbh, dtype, st);
    return run_group<ABFMT, false>(q, k, v, o, h, W, a, bh0, nbh, dtype, st);
}

// Backward of one group of slices in the same two passes (the parallel backward at head dimensions above 256):
//   pass 1 twice   Wn[r, c] = (q_r . k_c) e[r, c]            e[r, c] = exp2(gB_r + ga_c) = decay * scale / n_r
//                  dT[r, c] = (dh_r . v_c + g_r) e[r, c]     (c <= r; g_r = db_r n_r, gates.cu)
//   pass 2 thrice  dQ = dT K          (rows dotted with q: R)
//                  dK = dT^T Q        (rows dotted with k: dI)       contraction over the matrix rows (TRANS)
//                  dV = Wn^T dH
// Five contractions, the algorithmic minimum; the two matrices stay in L2 at moderate S.
template <int ABFMT, bool PAIR>
int run_group_bwd(const ScanGemmBwdArgs& a, int bh0, int nbh, int dtype, cudaStream_t st) {
    const size_t es = dtype == MLSTM_DT_F32 ? 4 : 2;
    const size_t slice = static_cast<size_t>(a.S) * a.D;
    auto at = [&](const void* base) { return static_cast<const uint8_t*>(base) + bh0 * slice * es; };
    auto at_out = [&](void* base) { return static_cast<uint8_t*>(base) + bh0 * slice * es; };
    GemmParams p{};
    p.S = a.S; p.Spad = a.Spad; p.BH = nbh; p.D = a.D;
    p.NT = a.Spad / TILE;
    p.NP = (p.NT + 1) / 2;
    p.NKT = (a.Spad + TN - 1) / TN;
    p.NVS = a.D / TN;
    p.per_head = 0;
    if (PAIR) for (int g = 0; g < p.NP; g++) p.per_head += g + 1;
    else for (int qt = 0; qt < p.NT; qt++) p.per_head += qt / 2 + 1;
    const size_t vec0 = static_cast<size_t>(bh0) * a.Spad, ref0 = static_cast<size_t>(bh0) * (a.Spad / REF_BLOCK);
    p.row_rel = a.gB + vec0; p.row_ref = a.An_ref + ref0;
    p.col_rel = a.ga + vec0; p.col_w = a.gaw + vec0; p.col_ref = a.a_ref + ref0;
    p.er_add = 0.0f;   // the scale is part of gB
    p.status = a.status;
    p.dot_stride = a.dot_stride;
    constexpr int KC = ABFMT == 2 ? 32 : 64;
    constexpr int GROUPS = TN * (ABFMT == 2 ? 4 : 2) / 128;
    constexpr int AT_GROUPS = TILE * (ABFMT == 2 ? 4 : 2) / 128;
    int rc;
    CUtensorMap ma, mb, mo, mg;
    int launch = 0;
    auto counter = [&]() { p.counter = a.counters + launch++; };
    const bool zero_counters = bh0 > 0;   // the gate pass cleared the five counters with the status word for the first group
    // ---- pass 1: Wn = gate(Q K^T), dT = gate(dH V^T + g)
    p.items = p.per_head * nbh;
    if ((rc = tc_make_map(&ma, at(a.q), nbh, a.S, a.D, dtype, false, 128)) != MLSTM_OK) return rc;
    if ((rc = tc_make_map(&mb, at(a.k), nbh, a.S, a.D, dtype, false, PAIR ? TN / 2 : TN)) != MLSTM_OK) return rc;
    if ((rc = tc_make_map_out(&mo, a.Wn, nbh, a.Spad, a.Spad, dtype, 32)) != MLSTM_OK) return rc;
    counter();
    if ((rc = launch_gemm<GATE, ABFMT, PAIR>(ma, mb, mo, mo, p, zero_counters, st)) != MLSTM_OK) return rc;
    p.row_g = a.g + vec0;
    if ((rc = tc_make_map(&ma, at(a.dh), nbh, a.S, a.D, dtype, false, 128)) != MLSTM_OK) return rc;
    if ((rc = tc_make_map(&mb, at(a.v), nbh, a.S, a.D, dtype, false, PAIR ? TN / 2 : TN)) != MLSTM_OK) return rc;
    if ((rc = tc_make_map_out(&mo, a.dT, nbh, a.Spad, a.Spad, dtype, 32)) != MLSTM_OK) return rc;
    counter();
    if ((rc = launch_gemm<GATE, ABFMT, PAIR>(ma, mb, mo, mo, p, zero_counters, st)) != MLSTM_OK) return rc;
    p.row_g = nullptr;
    // ---- pass 2
    p.items = (PAIR ? p.NP : p.NT) * nbh * p.NVS;
    // dQ = dT K, R = q . dQ
    p.side = SIDE_DOT;
    p.dot_out = a.R + vec0;
    if ((rc = tc_make_map(&ma, a.dT, nbh, a.Spad, a.Spad, dtype, false, 128)) != MLSTM_OK) return rc;
    if ((rc = tc_make_map_groups(&mb, at(a.k), nbh, a.S, a.D, dtype, ABFMT == 2, KC, PAIR ? GROUPS / 2 : GROUPS)) != MLSTM_OK) return rc;
    if ((rc = tc_make_map_out(&mo, at_out(a.dq), nbh, a.S, a.D, dtype, 32)) != MLSTM_OK) return rc;
    if ((rc = tc_make_map(&mg, at(a.q), nbh, a.S, a.D, dtype, false, 32)) != MLSTM_OK) return rc;
    counter();
    if ((rc = launch_gemm<APPLY, ABFMT, PAIR, false, true>(ma, mb, mo, mg, p, zero_counters, st)) != MLSTM_OK) return rc;
    // dK = dT^T Q, dI = k . dK
    p.dot_out = a.dI + vec0;
    if ((rc = tc_make_map_groups(&ma, a.dT, nbh, a.Spad, a.Spad, dtype, ABFMT == 2, KC, AT_GROUPS)) != MLSTM_OK) return rc;
    if ((rc = tc_make_map_groups(&mb, at(a.q), nbh, a.S, a.D, dtype, ABFMT == 2, KC, PAIR ? GROUPS / 2 : GROUPS)) != MLSTM_OK) return rc;
    if ((rc = tc_make_map_out(&mo, at_out(a.dk), nbh, a.S, a.D, dtype, 32)) != MLSTM_OK) return rc;
    if ((rc = tc_make_map(&mg, at(a.k), nbh, a.S, a.D, dtype, false, 32)) != MLSTM_OK) return rc;
    counter();
    if ((rc = launch_gemm<APPLY, ABFMT, PAIR, true, true>(ma, mb, mo, mg, p, zero_counters, st)) != MLSTM_OK) return rc;
    // dV = Wn^T dH
    p.side = SIDE_NONE;
    p.dot_out = nullptr;
    if ((rc = tc_make_map_groups(&ma, a.Wn, nbh, a.Spad, a.Spad, dtype, ABFMT == 2, KC, AT_GROUPS)) != MLSTM_OK) return rc;
    if ((rc = tc_make_map_groups(&mb, at(a.dh), nbh, a.S, a.D, dtype, ABFMT == 2, KC, PAIR ? GROUPS / 2 : GROUPS)) != MLSTM_OK) return rc;
    if ((rc = tc_make_map_out(&mo, at_out(a.dv), nbh, a.S, a.D, dtype, 32)) != MLSTM_OK) return rc;
    counter();
    return launch_gemm<APPLY, ABFMT, PAIR, true, true>(ma, mb, mo, mo, p, zero_counters, st);
}

template <int ABFMT>
int run_group_bwd_any(const ScanGemmBwdArgs& a, int bh0, int nbh, int dtype, cudaStream_t st) {
    if (use_pairs(a.Spad)) return run_group_bwd<ABFMT, true>(a, bh0, nbh, dtype, st);
    return run_group_bwd<ABFMT, false>(a, bh0, nbh, dtype, st);
}

}  // namespace

bool scan_gemm_supported(int S, int D, int in_dtype) {
    return S >= 1 && D > 256 && D % TN == 0 && D <= 4096 &&
           (in_dtype == MLSTM_DT_F16 || in_dtype == MLSTM_DT_BF16 || in_dtype == MLSTM_DT_F32);
}

// Slices whose gated matrices fit the budget at once (at least one): the passes run group by group.
int scan_gemm_group(int BH, int S, int dtype) {
    const size_t Spad = round_up(S, TILE);
    const size_t per_head = Spad * Spad * (dtype == MLSTM_DT_F32 ? 4 : 2);
    const size_t budget = static_cast<size_t>(512) << 20;
    size_t g = budget / per_head;
    if (g < 1) g = 1;
    return static_cast<int>(g < static_cast<size_t>(BH) ? g : BH);
}

size_t scan_gemm_w_bytes(int BH, int S, int dtype) {
    const size_t Spad = round_up(S, TILE);
    return static_cast<size_t>(scan_gemm_group(BH, S, dtype)) * Spad * Spad * (dtype == MLSTM_DT_F32 ? 4 : 2);
}

// The backward keeps two gated matrices per slice: half as many slices per group.
int scan_gemm_bwd_group(int BH, int S, int dtype) {
    const size_t Spad = round_up(S, TILE);
    const size_t per_head = 2 * Spad * Spad * (dtype == MLSTM_DT_F32 ? 4 : 2);
    const size_t budget = static_cast<size_t>(512) << 20;
    size_t g = budget / per_head;
    if (g < 1) g = 1;
    return static_cast<int>(g < static_cast<size_t>(BH) ? g : BH);
}

size_t scan_gemm_bwd_matrix_bytes(int BH, int S, int dtype) {   // one of the two matrices
    const size_t Spad = round_up(S, TILE);
    return static_cast<size_t>(scan_gemm_bwd_group(BH, S, dtype)) * Spad * Spad * (dtype == MLSTM_DT_F32 ? 4 : 2);
}

int launch_scan_gemm_bwd(const ScanGemmBwdArgs& a, int dtype, cudaStream_t st) {
    if (!scan_gemm_supported(a.S, a.D, dtype)) return MLSTM_E_UNSUPPORTED;
    const int group = scan_gemm_bwd_group(a.BH, a.S, dtype);
    for (int bh0 = 0; bh0 < a.BH; bh0 += group) {
        const int nbh = a.BH - bh0 < group ? a.BH - bh0 : group;
        int rc;
        switch (dtype) {
            case MLSTM_DT_F32: rc = run_group_bwd_any<2>(a, bh0, nbh, dtype, st); break;
            case MLSTM_DT_BF16: rc = run_group_bwd_any<1>(a, bh0, nbh, dtype, st); break;
            case MLSTM_DT_F16: rc = run_group_bwd_any<0>(a, bh0, nbh, dtype, st); break;
            default: return MLSTM_E_ARG;
        }
        if (rc != MLSTM_OK) return rc;
    }
    return MLSTM_OK;
}

size_t scan_gemm_bpart_bytes(int BH, int S, int dtype) {
    const size_t Spad = round_up(S, TILE);
    return static_cast<size_t>(scan_gemm_group(BH, S, dtype)) * ((Spad + TN - 1) / TN) * (nepi(GATE) / 4) * Spad * sizeof(float);
}

int launch_scan_gemm(const void* q, const void* k, const void* v, const void* o, float* h, void* W, const ScanGemmArgs& a,
                     int dtype, cudaStream_t st) {
    if (!scan_gemm_supported(a.S, a.D, dtype)) return MLSTM_E_UNSUPPORTED;
    const int group = scan_gemm_group(a.BH, a.S, dtype);
    for (int bh0 = 0; bh0 < a.BH; bh0 += group) {
        const int nbh = a.BH - bh0 < group ? a.BH - bh0 : group;
        int rc;
        switch (dtype) {
            case MLSTM_DT_F32: rc = run_group_any<2>(q, k, v, o, h, W, a, bh0, nbh, dtype, st); break;
            case MLSTM_DT_BF16: rc = run_group_any<1>(q, k, v, o, h, W, a, bh0, nbh, dtype, st); break;
            case MLSTM_DT_F16: rc = run_group_any<0>(q, k, v, o, h, W, a, bh0, nbh, dtype, st); break;
            default: return MLSTM_E_ARG;
        }
        if (rc != MLSTM_OK) return rc;
    }
    return MLSTM_OK;
}

}  // namespace mlstm
