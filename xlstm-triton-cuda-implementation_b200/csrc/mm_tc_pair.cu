// Tensor-core contraction pass on CTA PAIRS for the head dimension 256 (16-bit inputs): the same four
// passes and the same algebra as mm_tc.cu (see there and mlstm_common.cuh), with two CTAs of a
// cluster working on two neighbouring stationary tiles of one slice and sharing every streamed tile.
//
// Why: at D = 256 a single CTA streams 128 KB per step through the 160 KB that remain beside its
// stationary tile, so barely more than one step of loads can be in flight, and both operands of the
// first contraction come from shared memory at exactly its bandwidth.  With tcgen05.mma.cta_group::2
// one thread of the leader CTA issues M = 256 MMAs that run on both SMs: each CTA supplies its own 128
// rows of A (its stationary tile, or its W tile in TMEM) and HALF of B (64 of the 128 rows of the
// streamed Y tile for T = X Y^T; 128 of the 256 columns of the streamed Z tile for ACC += W Z), and
// gets its 128 rows of the result in its own TMEM.  Every CTA therefore loads 64 KB per step instead
// of 128 KB, the ring (4 x 32 KB) holds two steps, and 32 KB are left for staging the output tiles of
// TMA stores.  Measured at B=16, NH=8, S=4096, D=256, bf16: forward 0.84 ms against 0.98 ms for the
// one-CTA kernel, backward 2.8 ms against 3.2 ms.
//
// Signals that cross the pair every step (a gate warp's "W written" / "accumulator drained" arrival on
// the leader's barrier) use the default CTA-scope release: what they guard is TMEM, ordered by tcgen05
// fences.  With a cluster-scope release each arrival first waited for all of the thread's earlier
// memory operations to be visible cluster-wide and took over a thousand cycles.  Only the work-item ring
// (an ordinary shared-memory word written remotely, once per item) uses cluster-scope release/acquire.
//
// Roles per CTA as in mm_tc.cu (TMA producer warp, MMA warp, four gate groups); only the leader's MMA
// warp issues MMAs.  Barriers that the MMA thread waits on live in the leader (slot full, X loaded,
// W written, accumulator drained: the follower's TMA loads and gate warps signal them remotely);
// barriers that the MMA thread signals exist in both CTAs and get one tcgen05.commit each.  Every CTA
// issues its own loads into its own shared memory.  Every wait is bounded as in mm_tc.cu; the two hardware cluster barriers
// (after initialisation, before exit) are reached by every thread on every path.
#include <atomic>
#include <type_traits>

#include "mlstm_common.cuh"
#include "ptx_sm100.cuh"
#include "tc_host.cuh"

namespace mlstm {
namespace {

using namespace ptx;

constexpr int D = 256;
constexpr int NGROUPS = 4;
constexpr int NGATE = NGROUPS * 128;
constexpr int NTHREADS = 64 + NGATE;
constexpr int BOX_BYTES = 128 * 128;           // 128 rows x 128 bytes
constexpr int HBOX_BYTES = 64 * 128;           // 64 rows x 128 bytes (half of a streamed Y tile's rows)
constexpr int X_BYTES = (D / 64) * BOX_BYTES;  // 64 KB stationary tile
constexpr int SLOT_BYTES = 32 * 1024;          // Y half: 64 rows x 256 cols; Z half: 128 rows x 128 cols
constexpr int NSLOT = 4;                       // two steps of streamed tiles
constexpr int STAGE_BYTES = 2048;              // per gate warp: 32 rows x 64 bytes of output on their way to a TMA store
constexpr int OUT_BYTES = (NGATE / 32) * STAGE_BYTES;
constexpr int NBAR = 1 + 2 * NSLOT + 2 + 2 + 1 + 1 + 2 + 4 + 4;
constexpr int SMEM_BYTES = X_BYTES + NSLOT * SLOT_BYTES + OUT_BYTES + NBAR * 8 + 64 + NGROUPS * 128 * 4;
constexpr long long WAIT_LIMIT = 4000000000LL;
constexpr float MAX_ROW_EXP2 = 60.0f;           // clamp of the per-row exponent off the diagonal tile (see its use)
constexpr int SLACK_SLEEP_NS = 64;              // poll interval of the roles that wait with slack (gate warps, producer)
static_assert(SMEM_BYTES <= 232448, "exceeds the shared memory of a CTA");


template <int MODE, int ABFMT, typename OutT>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(NTHREADS, 1)
mlstm_tc_pass_pair(const __grid_constant__ CUtensorMap tmX, const __grid_constant__ CUtensorMap tmYh,
                   const __grid_constant__ CUtensorMap tmZ, const __grid_constant__ CUtensorMap tmO, const PassParams p) {
    using InT = typename std::conditional<ABFMT == 1, __nv_bfloat16, __half>::type;
    constexpr bool ROWS_ARE_Q = (MODE == FWD || MODE == DQ);
    constexpr bool IS_FWD = (MODE == FWD);

    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t* smem = smem_raw;
    uint8_t* sX = smem;
    uint8_t* sSlot = smem + X_BYTES;
    uint8_t* sOut = sSlot + NSLOT * SLOT_BYTES;
    uint64_t* bars = reinterpret_cast<uint64_t*>(sOut + OUT_BYTES);
    uint64_t* bar_x = bars;                     // leader: both stationary tiles loaded
    uint64_t* bar_full = bars + 1;              // leader: both halves of a slot loaded
    uint64_t* bar_empty = bars + 1 + NSLOT;     // both: slot no longer read by MMAs
    uint64_t* bar_t = bars + 1 + 2 * NSLOT;     // both [2]: T tile written
    uint64_t* bar_w = bar_t + 2;                // leader [2]: W tiles of both CTAs written (32 warp arrivals)
    uint64_t* bar_acc = bar_w + 2;              // both: accumulators complete
    uint64_t* bar_part = bar_acc + 1;           // own: row partials exchanged
    uint64_t* bar_xfree = bar_part + 1;         // both: stationary tiles no longer read
    uint64_t* bar_accfree = bar_xfree + 1;      // leader: accumulators of both CTAs drained (32 warp arrivals)
    uint64_t* bar_item = bar_accfree + 1;       // both [4]: work item published inside the CTA (by its own producer)
    uint64_t* bar_item_in = bar_item + 4;       // follower [4]: work item arrived from the leader's producer
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + NBAR);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    volatile int* item_ids = reinterpret_cast<volatile int*>(tmem_slot + 2);   // [4] ring read by this CTA's roles
    volatile int* item_in = reinterpret_cast<volatile int*>(tmem_slot + 6);    // [4] ring written by the leader (follower only)
    float* part = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(bars) + NBAR * 8 + 64);  // [NGROUPS][128]

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();    // 0 = leader
    const uint32_t peer = rank ^ 1u;
    const int NT = p.Spad / TILE;
    const int NP = (NT + 1) / 2;                 // tile pairs per slice
    const int total = NP * p.BH;
    const bool misaligned = (smem_u32(smem) & 1023u) != 0;   // uniform over the cluster in practice; never seen

    struct Item {
        int bh, pair, tile, nsteps;
    };
    auto decode = [&](int id) {
        Item it;
        const int SLICE_SET = p.slice_set;
        const int per_set = NP * SLICE_SET;
        const int set = id / per_set;
        const int within = id - set * per_set;
        const int set_size = min(SLICE_SET, p.BH - set * SLICE_SET);
        const int w = within / set_size;
        it.bh = set * SLICE_SET + (within - w * set_size);
        it.pair = ROWS_ARE_Q ? (NP - 1 - w) : w;           // heaviest first
        it.tile = 2 * it.pair + static_cast<int>(rank);     // this CTA's stationary tile (may be == NT: idle half)
        it.nsteps = ROWS_ARE_Q ? min(2 * it.pair + 2, NT) : (NT - 2 * it.pair);
        return it;
    };
    auto stream_tile = [&](const Item& it, int t) { return ROWS_ARE_Q ? t : (2 * it.pair + t); };

    // shared::cluster addresses of the leader's and the peer's copies of a barrier
    auto at_leader = [&](const void* local) { return mapa_u32(smem_u32(local), 0u); };
    auto at_peer = [&](const void* local) { return mapa_u32(smem_u32(local), peer); };

    if (threadIdx.x == 0) {
        mbar_init(bar_x, 1);
        mbar_init(bar_xfree, 1);
        for (int s = 0; s < NSLOT; s++) {
            mbar_init(&bar_full[s], 1);
            mbar_init(&bar_empty[s], 1);
        }
        mbar_init(&bar_t[0], 1);
        mbar_init(&bar_t[1], 1);
        mbar_init(&bar_w[0], 2 * NGATE / 32);
        mbar_init(&bar_w[1], 2 * NGATE / 32);
        mbar_init(bar_acc, 1);
        mbar_init(bar_accfree, 2 * NGATE / 32);
        mbar_init(bar_part, NGATE / 32);
        for (int k = 0; k < 4; k++) {
            mbar_init(&bar_item[k], 1);
            mbar_init(&bar_item_in[k], 1);
        }
        *abort_flag = misaligned ? 1 : 0;
        fence_mbar_init();
    }
    if (warp == 1) {
        tmem_alloc_pair(tmem_slot, 512);
        tmem_relinquish_pair();
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();           // the peer's barriers are initialised before anything signals them
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t tmem_T0 = tmem_base;
    const uint32_t tmem_ACC = tmem_base + 256;
    // nothing above touched global memory (see grid_dep_wait in mlstm_common.cuh)
    grid_dep_wait();
    grid_dep_launch();

    // Work items cross the pair once, from the leader's producer to the follower's (an ordinary shared-memory word
    // written remotely: cluster-scope release / acquire, which costs a thousand cycles and more); each producer
    // then publishes the item inside its own CTA, where the other roles get it with CTA-scope waits.
    auto next_item_warp = [&](int n, bool& ok) {   // gate warps (converged)
        ok = mbar_wait_warp<SLACK_SLEEP_NS>(&bar_item[n & 3], (n >> 2) & 1, abort_flag, WAIT_LIMIT);
        return ok ? __shfl_sync(0xffffffffu, item_ids[n & 3], 0) : -1;
    };

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer (one per CTA)
        if (lane == 0) {
            prefetch_tmap(&tmX);
            prefetch_tmap(&tmYh);
            prefetch_tmap(&tmZ);
            int slot_it = 0;
            bool ok = !*abort_flag;
            const uint32_t lead_x = at_leader(bar_x);
            for (int n = 0; ok; n++) {
                int id;
                if (rank == 0) {
                    id = atomicAdd(p.sched + MODE, 1);
                    if (id >= total) id = -1;
                    st_cluster_u32(at_peer(const_cast<int*>(&item_in[n & 3])), static_cast<uint32_t>(id));
                    mbar_arrive_cluster(at_peer(&bar_item_in[n & 3]));   // release at cluster scope: the peer sees the id
                } else {
                    ok = mbar_wait_cluster<SLACK_SLEEP_NS>(&bar_item_in[n & 3], (n >> 2) & 1, abort_flag, WAIT_LIMIT);
                    id = ok ? item_in[n & 3] : -1;
                }
                item_ids[n & 3] = id;
                mbar_arrive(&bar_item[n & 3]);   // CTA-scope release: this CTA's roles see the id
                if (id < 0) break;
                const Item it = decode(id);
                ok = mbar_wait<SLACK_SLEEP_NS>(bar_xfree, (n & 1) ^ 1, abort_flag, WAIT_LIMIT);
                if (!ok) break;
                if (rank == 0) mbar_expect_tx(bar_x, 2 * X_BYTES);
                for (int c = 0; c < D / 64; c++)   // rows past the end of the slice (idle half, ragged S) read as zeros
                    tma_load_3d_pair(sX + c * BOX_BYTES, &tmX, lead_x, c * 64, it.tile * TILE, it.bh);
                auto load_y = [&](int t) {   // this CTA's 64 rows of the streamed tile, all 256 columns
                    const int s = slot_it % NSLOT;
                    ok = ok && mbar_wait<SLACK_SLEEP_NS>(&bar_empty[s], ((slot_it / NSLOT) & 1) ^ 1, abort_flag, WAIT_LIMIT);
                    if (!ok) return;
                    if (rank == 0) mbar_expect_tx(&bar_full[s], 2 * SLOT_BYTES);
                    const uint32_t lead_full = at_leader(&bar_full[s]);
                    uint8_t* dst = sSlot + s * SLOT_BYTES;
                    const int row = stream_tile(it, t) * TILE + static_cast<int>(rank) * 64;
                    for (int c = 0; c < D / 64; c++) tma_load_3d_pair(dst + c * HBOX_BYTES, &tmYh, lead_full, c * 64, row, it.bh);
                    slot_it++;
                };
                auto load_z = [&](int t) {   // all 128 rows of the streamed tile, this CTA's 128 columns
                    const int s = slot_it % NSLOT;
                    ok = ok && mbar_wait<SLACK_SLEEP_NS>(&bar_empty[s], ((slot_it / NSLOT) & 1) ^ 1, abort_flag, WAIT_LIMIT);
                    if (!ok) return;
                    if (rank == 0) mbar_expect_tx(&bar_full[s], 2 * SLOT_BYTES);
                    const uint32_t lead_full = at_leader(&bar_full[s]);
                    uint8_t* dst = sSlot + s * SLOT_BYTES;
                    for (int c = 0; c < 2; c++)
                        tma_load_3d_pair(dst + c * BOX_BYTES, &tmZ, lead_full, static_cast<int>(rank) * 128 + c * 64,
                                         stream_tile(it, t) * TILE, it.bh);
                    slot_it++;
                };
                load_y(0);
                for (int t = 1; t < it.nsteps && ok; t++) {
                    load_y(t);
                    load_z(t - 1);
                }
                if (ok) load_z(it.nsteps - 1);
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer (leader only)
        // the whole warp runs the loop, one elected lane issues (see mm_tc.cu for why)
        if (rank == 0) {
            const bool issuer = elect_one();
            auto uni = [](int x) { return __shfl_sync(0xffffffffu, x, 0); };
            auto wait_u = [&](uint64_t* bar, uint32_t parity) { return mbar_wait_warp(bar, parity, abort_flag, WAIT_LIMIT); };
            constexpr uint32_t idesc1 = make_idesc(ABFMT, 256, 128, 0, 0);
            constexpr uint32_t idesc2 = make_idesc(ABFMT, 256, 256, 0, 1);
            const uint32_t sX_u = static_cast<uint32_t>(uni(static_cast<int>(smem_u32(sX))));
            const uint32_t sSlot_u = sX_u + X_BYTES;
            const uint32_t bars_u = sSlot_u + NSLOT * SLOT_BYTES + OUT_BYTES;   // this CTA's barriers ...
            const uint32_t bars_peer_u = static_cast<uint32_t>(uni(static_cast<int>(at_peer(bars))));   // ... and the peer's
            const uint32_t tmem_T0u = static_cast<uint32_t>(uni(static_cast<int>(tmem_T0)));
            const uint32_t tmem_ACCu = tmem_T0u + 256;
            const uint64_t xdesc0 = smem_desc_sw128(sX_u, 16, 1024);
            const uint64_t ydesc0 = smem_desc_sw128(sSlot_u, 16, 1024);
            const uint64_t zdesc0 = smem_desc_sw128(sSlot_u, BOX_BYTES, 1024, 2);
            auto commit_both = [&](const uint64_t* bar) {   // one arrival in either CTA
                const uint32_t off = static_cast<uint32_t>(bar - bars) * 8u;
                tc_commit_pair(bars_u + off);
                tc_commit_pair(bars_peer_u + off);
            };
            int slot_it = 0;
            int gstep = 0;
            bool ok = __all_sync(0xffffffffu, *abort_flag ? 0 : 1) != 0;
            for (int n = 0; ok; n++) {
                ok = wait_u(&bar_item[n & 3], (n >> 2) & 1);
                if (!ok) break;
                const int id = uni(item_ids[n & 3]);
                if (id < 0) break;
                const Item it = decode(id);
                ok = wait_u(bar_x, n & 1);
                if (!ok) break;
                tc_fence_after();
                auto second = [&](int u) {  // ACC += W(u) Z(u), both CTAs
                    const int gu = gstep + u;
                    ok = ok && wait_u(&bar_w[gu & 1], (gu >> 1) & 1);
                    if (ok && u == 0) ok = wait_u(bar_accfree, (n & 1) ^ 1);
                    if (!ok) return;
                    tc_fence_after();
                    const int s = slot_it % NSLOT;
                    ok = wait_u(&bar_full[s], (slot_it / NSLOT) & 1);
                    if (!ok) return;
                    const uint32_t w_tmem = tmem_T0u + (gu & 1) * 128;
                    const uint64_t zdesc = smem_desc_advance(zdesc0, s * SLOT_BYTES);
                    if (issuer) {
#pragma unroll
                        for (int kk = 0; kk < 8; kk++) {   // 16 streamed rows per MMA; N = 256 (128 columns from each CTA)
                            const uint32_t a_tmem = w_tmem + (kk >> 1) * 32 + (kk & 1) * 8;
                            mma_ts_pair(tmem_ACCu, a_tmem, smem_desc_advance(zdesc, kk * 2048), idesc2, (u > 0 || kk > 0) ? 1u : 0u);
                        }
                        commit_both(&bar_empty[s]);
                    }
                    __syncwarp();
                    slot_it++;
                };
                for (int t = 0; t < it.nsteps && ok; t++) {
                    const int gt = gstep + t;
                    const uint32_t t_tmem = tmem_T0u + (gt & 1) * 128;
                    const int s = slot_it % NSLOT;
                    ok = wait_u(&bar_full[s], (slot_it / NSLOT) & 1);
                    if (!ok) break;
                    const uint64_t ydesc = smem_desc_advance(ydesc0, s * SLOT_BYTES);
                    if (issuer) {
#pragma unroll
                        for (int kx = 0; kx < D / 16; kx++) {   // T(t) = X Y(t)^T: N = 128 (64 rows of Y from each CTA)
                            mma_ss_pair(t_tmem, smem_desc_advance(xdesc0, (kx >> 2) * BOX_BYTES + (kx & 3) * 32),
                                        smem_desc_advance(ydesc, (kx >> 2) * HBOX_BYTES + (kx & 3) * 32), idesc1, kx > 0 ? 1u : 0u);
                        }
                        commit_both(&bar_empty[s]);
                        commit_both(&bar_t[gt & 1]);
                        if (t == it.nsteps - 1) commit_both(bar_xfree);
                    }
                    __syncwarp();
                    slot_it++;
                    if (t >= 1) second(t - 1);
                }
                if (ok) second(it.nsteps - 1);
                if (ok && issuer) commit_both(bar_acc);
                __syncwarp();
                gstep += it.nsteps;
            }
        }
    } else {
        // ------------------------------------------------------------ gate groups
        const int grp = (warp - 2) >> 2;
        const int r = (warp & 3) * 32 + lane;
        const uint32_t lane_bits = static_cast<uint32_t>((warp & 3) * 32) << 16;
        const int cbase = grp * 32;
        auto load_cols = [&](const float* base, float (&dst)[32]) {
            const float4* p4 = reinterpret_cast<const float4*>(base + cbase);
#pragma unroll
            for (int q4 = 0; q4 < 8; q4++) {
                const float4 e4 = __ldg(p4 + q4);
                dst[q4 * 4 + 0] = e4.x; dst[q4 * 4 + 1] = e4.y; dst[q4 * 4 + 2] = e4.z; dst[q4 * 4 + 3] = e4.w;
            }
        };
        const uint32_t lead_w[2] = {at_leader(&bar_w[0]), at_leader(&bar_w[1])};
        const uint32_t lead_accfree = at_leader(bar_accfree);
        bool ok = __all_sync(0xffffffffu, *abort_flag == 0) != 0;
        int gstep = 0;
        uint8_t* stage = sOut + (warp - 2) * STAGE_BYTES;
        if (lane == 0) prefetch_tmap(&tmO);

        // Row terms of a work item: the row part of the exponent (a float relative to a double block reference,
        // added up in double) and the DQ additive term.  Fetching (the loads) and combining (the first use of what
        // was loaded) are separate steps: the next item's terms are requested before the accumulator wait of this
        // item and combined only when that item starts, so nobody waits for those loads.
        struct RowRaw {
            float rel, g;
            double ref;
        };
        auto fetch_rows = [&](const Item& it) {
            RowRaw rr{0.0f, 0.0f, 0.0};
            if (it.tile < NT) {
                const int grow = it.tile * TILE + r;
                const size_t vec_base = static_cast<size_t>(it.bh) * p.Spad;
                rr.rel = p.row_rel[vec_base + grow];
                rr.ref = p.row_ref[static_cast<size_t>(it.bh) * (p.Spad / REF_BLOCK) + grow / REF_BLOCK];
                if (MODE == DQ) rr.g = p.row_g[vec_base + grow];
            }
            return rr;
        };
        constexpr int UNKNOWN = -2;
        int id = next_item_warp(0, ok);
        RowRaw raw{0.0f, 0.0f, 0.0};
        if (ok && id >= 0) raw = fetch_rows(decode(id));

        for (int n = 0; ok && id >= 0; n++) {
        const Item it = decode(id);
        const int bh = it.bh, tile = it.tile, nsteps = it.nsteps;
        const bool active = tile < NT;                 // the idle half of an odd last pair only keeps the protocol going
        const int grow = tile * TILE + r;
        const size_t vec_base = static_cast<size_t>(bh) * p.Spad;
        const size_t ref_base = static_cast<size_t>(bh) * (p.Spad / REF_BLOCK);
        const double er_d = active ? static_cast<double>(raw.rel) + raw.ref + static_cast<double>(p.er_add) : 0.0;
        const float g_row = raw.g;
        float rowsum = 0.0f;

        for (int t = 0; t < nsteps; t++) {
            const int gt = gstep + t;
            const int buf = gt & 1;
            const int st = stream_tile(it, t);
            const bool diag = (st == tile);
            // tiles on the wrong side of this CTA's diagonal (they belong to the partner's triangle) give W = 0
            const bool dead = !active || (ROWS_ARE_Q ? (st > tile) : (st < tile));
            float cv[32];
            if (!dead) load_cols((diag ? p.col_rel : p.col_w) + vec_base + st * TILE, cv);
            const float er = dead ? 0.0f : static_cast<float>(er_d + p.col_ref[ref_base + st * (TILE / REF_BLOCK) + (grp >> 1)]);
            // DK adds a per-column term to T.  Each lane fetches one column's value before the wait (32 more
            // registers are not to be had) and the warp passes them round with shuffles afterwards.
            const float g_lane = (MODE == DK && !dead) ? __ldg(p.col_g + vec_base + st * TILE + cbase + lane) : 0.0f;
            ok = mbar_wait_warp<SLACK_SLEEP_NS>(&bar_t[buf], (gt >> 1) & 1, abort_flag, WAIT_LIMIT);
            if (!ok) break;
            tc_fence_after();
            const uint32_t t_tmem = tmem_T0 + buf * 128 + lane_bits + cbase;
            uint32_t pk[16];
            if (dead) {
#pragma unroll
                for (int j = 0; j < 16; j++) pk[j] = 0u;
            } else {
                uint32_t tv[32];
                tmem_ld32(t_tmem, tv);
                tc_wait_ld();
                if (MODE == DK) {
#pragma unroll
                    for (int j = 0; j < 32; j++)
                        tv[j] = __float_as_uint(__uint_as_float(tv[j]) + __shfl_sync(0xffffffffu, g_lane, j));
                }
                if (diag) {
#pragma unroll
                    for (int j = 0; j < 32; j++) {
                        float tval = __uint_as_float(tv[j]);
                        if (MODE == DQ) tval += g_row;
                        float wj = tval * fast_exp2(cv[j] + er);
                        if (!causal_ok<MODE>(r, cbase + j)) wj = 0.0f;
                        if (IS_FWD) rowsum += wj;
                        cv[j] = wj;
                    }
                } else {
                    // A 64-column block that is padding from end to end (ragged S) has no meaningful reference, and the
                    // row term alone can be large with strong decay: its column factors are 0, and 0 times an overflowed
                    // u would be NaN.  Real columns keep er far below the clamp.
                    const float u = fast_exp2(fminf(er, MAX_ROW_EXP2));
                    const float gu = (MODE == DQ) ? g_row * u : 0.0f;
#pragma unroll
                    for (int j = 0; j < 32; j++) {
                        const float tu = (MODE == DQ) ? fmaf(__uint_as_float(tv[j]), u, gu) : __uint_as_float(tv[j]) * u;
                        const float wj = tu * cv[j];
                        if (IS_FWD) rowsum += wj;
                        cv[j] = wj;
                    }
                }
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
            }
            tmem_st16(t_tmem, pk);
            tc_wait_st();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_remote(lead_w[buf]);
        }
        if (!ok) break;
        gstep += nsteps;

        // ---- while the last contractions run: everything of the epilogue that does not need the accumulator
        const bool row_ok = active && (grow < p.S);
        float inv_n = 1.0f;
        auto exchange = [&](float x) {   // sum of one value per gate group for this row
            part[grp * 128 + r] = x;
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_part);
            ok = mbar_wait_warp<SLACK_SLEEP_NS>(bar_part, n & 1, abort_flag, WAIT_LIMIT);
            return ok ? (part[r] + part[128 + r]) + (part[256 + r] + part[384 + r]) : 0.0f;
        };
        auto fwd_norm = [&]() {
            const float mrow = row_ok ? p.m[static_cast<size_t>(bh) * p.S + grow] : 0.0f;   // on its way during the exchange
            const float bsum = exchange(rowsum);
            if (ok) {
                inv_n = 1.0f / (fmaxf(fabsf(bsum), __expf(-mrow)) + 1e-6f);
                if (grp == 0 && row_ok && p.b_out) p.b_out[static_cast<size_t>(bh) * p.S + grow] = bsum;
            }
        };
        // The row partials are reused from item to item.  Nobody still reads the previous item's: a warp gets
        // past step 2 of this item only after every gate warp of the pair has finished step 0 of it (the third
        // T tile follows the first W tile), which follows its previous epilogue.  Shorter items exchange later.
        if (IS_FWD && nsteps > 2) fwd_norm();
        if (!ok) break;
        // next work item, if it is published already, and its row terms
        int id_next = UNKNOWN;
        RowRaw raw_next{0.0f, 0.0f, 0.0};
        if (__all_sync(0xffffffffu, mbar_test_wait(&bar_item[(n + 1) & 3], ((n + 1) >> 2) & 1) ? 1 : 0)) {
            id_next = __shfl_sync(0xffffffffu, item_ids[(n + 1) & 3], 0);
            if (id_next >= 0) raw_next = fetch_rows(decode(id_next));
        }

        // DQ / DK: the operand of the epilogue's row dot (this thread's 64 values of q resp. k: one 128-byte line) is
        // read by no other part of the pass, so it would come from DRAM after the accumulator wait; ask for it now
        if ((MODE == DQ || MODE == DK) && p.dot_src && row_ok)
            prefetch_l2(reinterpret_cast<const InT*>(p.dot_src) + (static_cast<size_t>(bh) * p.S + grow) * D + grp * (D / NGROUPS));
        // ---- epilogue: each group drains a quarter of this CTA's accumulator columns
        ok = mbar_wait_warp<SLACK_SLEEP_NS>(bar_acc, n & 1, abort_flag, WAIT_LIMIT);
        if (!ok) break;
        {
            tc_fence_after();
            constexpr int QUART = D / NGROUPS;   // 64
            const int c0 = grp * QUART;
            const size_t row_off = (static_cast<size_t>(bh) * p.S + (row_ok ? grow : 0)) * D;
            if (IS_FWD && nsteps <= 2) fwd_norm();
            if (!ok) break;
            float dot = 0.0f;
            const InT* ogate_row = (IS_FWD && p.ogate) ? reinterpret_cast<const InT*>(p.ogate) + row_off + c0 : nullptr;
            const InT* drow = ((MODE == DQ || MODE == DK) && p.dot_src) ? reinterpret_cast<const InT*>(p.dot_src) + row_off + c0
                                                                        : nullptr;
#pragma unroll 1
            for (int ch = 0; ch < QUART / 32; ch++) {
                uint32_t av[32];
                tmem_ld32(tmem_ACC + lane_bits + c0 + ch * 32, av);
                tc_wait_ld();
                if (ch == QUART / 32 - 1) {
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive_remote(lead_accfree);
                }
                float vals[32];
#pragma unroll
                for (int j = 0; j < 32; j++) vals[j] = __uint_as_float(av[j]) * inv_n;
                if (row_ok) {
                    if (IS_FWD && ogate_row) {
#pragma unroll
                        for (int j = 0; j < 32; j++) vals[j] *= silu_f(to_f32<InT>(ogate_row[ch * 32 + j]));
                    }
                    if ((MODE == DQ || MODE == DK) && drow) {
#pragma unroll
                        for (int jv = 0; jv < 4; jv++) {
                            const uint4 raw = *reinterpret_cast<const uint4*>(drow + ch * 32 + jv * 8);
                            const InT* ev = reinterpret_cast<const InT*>(&raw);
#pragma unroll
                            for (int j = 0; j < 8; j++) dot += vals[jv * 8 + j] * to_f32<InT>(ev[j]);
                        }
                    }
                }
                // This warp's 32 rows x 32 columns go out through its staging buffer and a TMA store (rows past
                // the end of the slice are not written): scattered 16-byte stores from registers took several
                // thousand cycles per item during which the tensor pipe had nothing to do.
                constexpr int NSUB = sizeof(OutT) == 4 ? 2 : 1;    // 64 bytes per row and store
#pragma unroll
                for (int sub = 0; sub < NSUB; sub++) {
                    if (lane == 0) bulk_wait_read_all();   // the previous store has read the buffer
                    __syncwarp();
                    uint4* srow = reinterpret_cast<uint4*>(stage + lane * 64);
                    const int sw = (lane >> 1) & 3;   // 64-byte swizzle of the store's tensor map: no bank conflicts
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
                    if (lane == 0 && active) {
                        tma_store_3d(&tmO, stage, c0 + ch * 32 + sub * (64 / static_cast<int>(sizeof(OutT))),
                                     tile * TILE + (warp & 3) * 32, bh);
                        bulk_commit();
                    }
                }
            }
            // one partial per gate group: adding them up is left to the dF kernel, so that the groups need not meet here
            if ((MODE == DQ || MODE == DK) && p.dot_out && active)
                p.dot_out[grp * p.dot_part_stride + vec_base + grow] = row_ok ? dot : 0.0f;
        }
        if (!ok) break;
        // ---- on to the next item
        if (id_next == UNKNOWN) {
            id_next = next_item_warp(n + 1, ok);
            if (ok && id_next >= 0) raw_next = fetch_rows(decode(id_next));
        }
        id = id_next;
        raw = raw_next;
        }  // items
        if (lane == 0) bulk_wait_all();   // the last stores have left shared memory before the CTA goes away
        tc_fence_before();
    }

    __syncthreads();
    if (*abort_flag) {
        if (threadIdx.x == 0) atomicExch(p.status, misaligned ? 2000 : 3000 + MODE);
        for (int k = 0; k < 64; k++) __nanosleep(16000);
        __syncthreads();
    }
    cluster_sync_all();   // neither CTA releases shared memory or TMEM the other may still touch
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc_pair(tmem_base, 512);
    }
}

template <int MODE, int ABFMT, typename OutT>
int launch_pair_one(const PassParams& p_in, int in_dtype, cudaStream_t st) {
    PassParams p = p_in;
    p.slice_set = tc_slice_set();
    CUtensorMap mx, myh, mz, mo;
    int rc;
    constexpr int out_dtype = sizeof(OutT) == 4 ? MLSTM_DT_F32 : (ABFMT == 1 ? MLSTM_DT_BF16 : MLSTM_DT_F16);
    if ((rc = tc_make_map_out(&mo, p.out, p.BH, p.S, D, out_dtype, 32)) != MLSTM_OK) return rc;
    if ((rc = tc_make_map(&mx, p.X, p.BH, p.S, D, in_dtype, false, 128)) != MLSTM_OK) return rc;
    if ((rc = tc_make_map(&myh, p.Y, p.BH, p.S, D, in_dtype, false, 64)) != MLSTM_OK) return rc;
    if ((rc = tc_make_map(&mz, p.Z, p.BH, p.S, D, in_dtype, false, 128)) != MLSTM_OK) return rc;
    auto kern = mlstm_tc_pass_pair<MODE, ABFMT, OutT>;
    // per device: shared-memory opt-in and how many pairs can be resident at once (both idempotent, so
    // concurrent first callers may both run the set-up; the count is published last)
    static std::atomic<int> pairs_resident_dev[64];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return MLSTM_E_CUDA;
    int pairs_resident = pairs_resident_dev[dev].load(std::memory_order_acquire);
    if (pairs_resident == 0) {
        cudaError_t ce = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
        if (ce != cudaSuccess) {
            cudaGetLastError();
            return note_cuda_error(ce, "cudaFuncSetAttribute(MaxDynamicSharedMemorySize)");
        }
        const int sms = tc_sm_count();
        if (sms <= 1) return MLSTM_E_CUDA;
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(static_cast<unsigned>(sms & ~1), 1, 1);
        cfg.blockDim = dim3(NTHREADS, 1, 1);
        cfg.dynamicSmemBytes = SMEM_BYTES;
        cudaLaunchAttribute attr;
        attr.id = cudaLaunchAttributeClusterDimension;
        attr.val.clusterDim.x = 2;
        attr.val.clusterDim.y = 1;
        attr.val.clusterDim.z = 1;
        cfg.attrs = &attr;
        cfg.numAttrs = 1;
        int nclusters = 0;
        ce = cudaOccupancyMaxActiveClusters(&nclusters, kern, &cfg);
        if (ce != cudaSuccess || nclusters <= 0) {
            cudaGetLastError();
            nclusters = sms / 2;   // the grid does not have to be resident at once: CTAs only wait inside their pair
        }
        pairs_resident = nclusters < sms / 2 ? nclusters : sms / 2;
        pairs_resident_dev[dev].store(pairs_resident, std::memory_order_release);
    }
    const int NT = p.Spad / TILE;
    const long long total = static_cast<long long>((NT + 1) / 2) * p.BH;
    if (total > 0x3fffffffLL) return MLSTM_E_SHAPE;
    const unsigned npairs = static_cast<unsigned>(total < pairs_resident ? total : pairs_resident);
    if (!p.sched) return MLSTM_E_ARG;
    cudaError_t ce = cudaSuccess;
    if (!p.sched_zeroed) {
        ce = cudaMemsetAsync(p.sched + MODE, 0, sizeof(int), st);
        if (ce != cudaSuccess) return note_cuda_error(ce, "cudaMemsetAsync(item counter)");
    }
    ce = launch_pdl(kern, dim3(2 * npairs), dim3(NTHREADS), SMEM_BYTES, st, mx, myh, mz, mo, p);
    if (ce != cudaSuccess) cudaGetLastError();
    return ce == cudaSuccess ? MLSTM_OK : note_cuda_error(ce, "launch of mlstm_tc_pass_pair");
}

template <int MODE>
int launch_pair_fmt(const PassParams& p, int in_dtype, int out_dtype, cudaStream_t st) {
    if (in_dtype == MLSTM_DT_BF16) {
        if (out_dtype == MLSTM_DT_F32) return launch_pair_one<MODE, 1, float>(p, in_dtype, st);
        if (out_dtype == in_dtype) return launch_pair_one<MODE, 1, __nv_bfloat16>(p, in_dtype, st);
    } else if (in_dtype == MLSTM_DT_F16) {
        if (out_dtype == MLSTM_DT_F32) return launch_pair_one<MODE, 0, float>(p, in_dtype, st);
        if (out_dtype == in_dtype) return launch_pair_one<MODE, 0, __half>(p, in_dtype, st);
    }
    return MLSTM_E_ARG;
}

}  // namespace


// 16-bit inputs, head dimension 256, at least two tiles per slice (a single tile has no partner)
bool tc_pair_supported(int S, int Dh, int in_dtype) {
    return S > TILE && Dh == 256 && (in_dtype == MLSTM_DT_F16 || in_dtype == MLSTM_DT_BF16);
}

int launch_pass_tc_pair(int mode, const PassParams& p, int in_dtype, int out_dtype, cudaStream_t st) {
    if (!tc_pair_supported(p.S, p.D, in_dtype)) return MLSTM_E_UNSUPPORTED;
    switch (mode) {
        case FWD: return launch_pair_fmt<FWD>(p, in_dtype, out_dtype, st);
        case DQ: return launch_pair_fmt<DQ>(p, in_dtype, out_dtype, st);
        case DK: return launch_pair_fmt<DK>(p, in_dtype, out_dtype, st);
        case DV: return launch_pair_fmt<DV>(p, in_dtype, out_dtype, st);
    }
    return MLSTM_E_UNSUPPORTED;
}

}  // namespace mlstm
