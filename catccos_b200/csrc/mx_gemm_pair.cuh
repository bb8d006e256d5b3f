// MXFP8 block-scaled GEMM on CTA pairs (clusters of two SMs, tcgen05 cta_group::2).
//
// Same operator, operands, layouts and flag gating as mx_gemm.cuh; what changes is the tile: a pair of
// CTAs owns a 256 x 256 output tile.  CTA r of the pair loads A rows [m0 + 128 r, +128) and B columns
// [n0 + 128 r, +128) of every K tile (32 KB per K tile per SM instead of 48 KB), the leader CTA (r = 0)
// issues one tcgen05.mma.cta_group::2 (M = 256, N = 256, K = 32) that reads both CTAs' shared memory, and
// each CTA ends up with the accumulator of its own 128 rows x 256 columns in its own tensor memory.
// Every CTA loads its own tiles with plain TMA (no cluster multicast anywhere); what crosses the pair is
// only barrier traffic:
//   full[s]                     lives in the leader; both CTAs' TMA bytes go there, and the commit behind the
//                               leader's scale copies (tcgen05.cp.cta_group::2 reads the atoms of both CTAs)
//   atoms_written[s]            lives in the leader; both CTAs' scale loaders arrive once their atoms are in
//                               shared memory
//   empty[s], tmem_full[a]      live in each CTA; the leader's tcgen05.commit arrives on both copies
//   tmem_empty[a], overlap_free[a]  live in the leader; the epilogue warps of both CTAs arrive there
#pragma once

#include "mx_gemm.cuh"

namespace catccos {

constexpr uint32_t kPairBlockM = 256;
constexpr uint32_t kPairBlockN = 256;

struct PairSmem {
    static constexpr uint32_t kStages = 5;
    static constexpr uint32_t kABytes = 128 * kGemmBlockK;  // this CTA's 128 rows
    static constexpr uint32_t kBBytes = 128 * kGemmBlockK;  // this CTA's 128 columns
    static constexpr uint32_t kSfaBytes = 512;
    static constexpr uint32_t kSfbBytes = 1024;  // all 256 columns: each CTA multiplies by the whole N tile
    static constexpr uint32_t kOffA = 0;
    static constexpr uint32_t kOffB = kOffA + kStages * kABytes;
    static constexpr uint32_t kOffSfa = kOffB + kStages * kBBytes;
    static constexpr uint32_t kOffSfb = kOffSfa + kStages * kSfaBytes;
    static constexpr uint32_t kOffBar = kOffSfb + kStages * kSfbBytes;
    // full[S], empty[S], tmem_full[2], tmem_empty[2], overlap_free[2], atoms_written[S] (leader only: both
    // CTAs' scale loaders have put a stage's atoms into shared memory)
    static constexpr uint32_t kNumBars = 3 * kStages + 6;
    static constexpr uint32_t kOffTmemPtr = kOffBar + kNumBars * 8;
    static constexpr uint32_t kOffGate = kOffTmemPtr + 8;  // K-tile iterations whose rows this CTA's producer has seen ready
    static constexpr uint32_t kBytes = kOffTmemPtr + 16;
    static constexpr uint32_t kDynamicBytes = kBytes + 1024;
    static constexpr uint32_t kOverlapChunks = 2;
    static constexpr uint32_t kAccCol1 = 192;  // the two accumulators share columns 192..255 (see mx_gemm.cuh)
    static constexpr uint32_t kSfCol = 448;    // one scale-factor set of 12 columns per stage
    static constexpr uint32_t kSfSetCols = 12;
    static_assert(kSfCol + kStages * kSfSetCols <= 512, "scale-factor sets must fit in tensor memory");
};

// Tile order for pairs: as tile_coord, with 256-row tiles.
__host__ __device__ __forceinline__ TileCoord pair_tile_coord(uint32_t idx, uint32_t n_tiles, uint32_t m_tiles, const GemmParams& p)
{
    uint32_t mo = idx / n_tiles;
    TileCoord t;
    t.n_tile = idx - mo * n_tiles;
    t.m_tile = mo;
    if (p.flags != nullptr && p.world > 1) {
        if (p.m_local % kPairBlockM == 0) {
            t.m_tile = arrival_m_tile(mo, p.m_local / kPairBlockM, p);
        } else {
            t.m_tile = (mo + (p.rank * p.m_local) / kPairBlockM) % m_tiles;
        }
    }
    return t;
}

template <typename OutT, bool FUSED_QUANT>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(FUSED_QUANT ? kGemmFusedThreads : kGemmThreads, 1)
mx_gemm_pair_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b, GemmParams p)
{
    using S = PairSmem;
    constexpr uint32_t kStages = S::kStages;

    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + S::kOffBar);
    uint64_t* full = bars;
    uint64_t* empty = bars + kStages;
    uint64_t* tmem_full = bars + 2 * kStages;
    uint64_t* tmem_empty = tmem_full + 2;
    uint64_t* overlap_free = tmem_empty + 2;
    uint64_t* atoms_written = overlap_free + 2;
    uint32_t* tmem_ptr_smem = reinterpret_cast<uint32_t*>(smem + S::kOffTmemPtr);
    uint32_t* gate = reinterpret_cast<uint32_t*>(smem + S::kOffGate);
    uint32_t* push_turn = gate + 1;  // the pushers of this CTA store one after the other (mx_quant.cuh, push_worker)

    const uint32_t warp = threadIdx.x >> 5;
    const uint32_t lane = threadIdx.x & 31;
    const uint32_t cta = cluster_ctarank();  // 0 = leader
    const uint64_t bar_ns = p.bar_timeout_ns;
    const uint32_t pair = blockIdx.x >> 1;
    const uint32_t num_pairs = gridDim.x >> 1;

    const uint32_t m_tiles = (p.Mg + kPairBlockM - 1) / kPairBlockM;
    const uint32_t n_tiles = (p.N + kPairBlockN - 1) / kPairBlockN;
    const uint32_t num_tiles = p.gemm_off ? 0u : m_tiles * n_tiles;
    const uint32_t k_tiles = p.K / kGemmBlockK;

    if (threadIdx.x == 0) {
        CATCCOS_TR_STAMP(p.trace, kTrCtaStart);
        *gate = 0u;
        *push_turn = 0u;
        for (uint32_t s = 0; s < kStages; ++s) {
            mbar_init(&full[s], 3);  // both CTAs' producers (expect_tx) and the commit behind the scale copies
            mbar_init(&empty[s], 1);
            mbar_init(&atoms_written[s], 2);  // one scale-loader warp in each CTA
        }
        for (uint32_t a = 0; a < 2; ++a) {
            mbar_init(&tmem_full[a], 1);
            mbar_init(&tmem_empty[a], 8);    // four epilogue warps in each CTA
            mbar_init(&overlap_free[a], 8);
        }
        mbar_fence_init();
        tma_prefetch_desc(&tmap_a);
        tma_prefetch_desc(&tmap_b);
    }
    if (warp == 5) {
        tmem_alloc_pair(tmem_ptr_smem, kTmemCols);
        tmem_relinquish_pair();
    }
    tcgen05_fence_before();
    __syncthreads();
    cluster_sync_all();  // both CTAs' barriers exist before anybody arrives on the other's
    tcgen05_fence_after();
    const uint32_t tmem_base = *tmem_ptr_smem;

    if (threadIdx.x == 0) {
        CATCCOS_TR_STAMP(p.trace, kTrSetupDone);
    }

    if (warp == 4) {
        // ------------------------------- TMA producer (both CTAs) -------------------------
        if (p.flags == nullptr) {
            grid_dep_wait();  // A is the output of the kernel launched just before (no-op for a plain launch);
        }                     // with flags, the flags say when its rows are there
        uint32_t it = 0, ti = 0;
        bool alive = true;
        // packed 4-bit operands arrive as half the bytes they occupy in shared memory (the gaps are not written)
        const uint32_t tx_bytes = (p.a_fmt == 5u ? S::kABytes / 2u : S::kABytes) + (p.b_fmt == 5u ? S::kBBytes / 2u : S::kBBytes);
        for (uint32_t tile = pair; alive && tile < num_tiles; tile += num_pairs, ++ti) {
            TileCoord tc = pair_tile_coord(tile, n_tiles, m_tiles, p);
            const uint32_t m0 = tc.m_tile * kPairBlockM + cta * 128u;
            const uint32_t n0 = tc.n_tile * kPairBlockN + cta * 128u;
            uint32_t ready_end = 0;  // K tiles below this index are known to be there
            for (uint32_t kt = 0; alive && kt < k_tiles; ++kt, ++it) {
                if (p.flags != nullptr && kt >= ready_end) {
                    const unsigned long long t0 = CATCCOS_TR_NOW();
                    (void)t0;
                    const uint32_t seg0 = kt / p.seg_ktiles;
                    const uint32_t nready = wait_rows_ready(p, m0, lane, seg0);
                    alive = nready != 0u;
                    ready_end = min((seg0 + nready) * p.seg_ktiles, k_tiles);
                    fence_proxy_async_all();
                    if (lane == 0) {
                        st_release_cta_shared(gate, it + (ready_end - kt));
                        CATCCOS_TR_ADD(p.trace, kTrProdFlagWaitNs, CATCCOS_TR_NOW() - t0);
                    }
                }
                if (lane == 0 && alive) {
                    const uint32_t s = it % kStages;
                    const uint32_t ph = (it / kStages) & 1u;
                    const unsigned long long t1 = CATCCOS_TR_NOW();
                    (void)t1;
                    alive = mbar_wait_cluster(&empty[s], ph ^ 1u, p.status, 200, s, bar_ns);
                    CATCCOS_TR_ADD(p.trace, kTrProdEmptyWaitNs, CATCCOS_TR_NOW() - t1);
                    if (kt == 0 && ti < kTraceTiles) {
                        CATCCOS_TR_STAMP(p.trace, kTrTileStart + ti);
                    }
                    CATCCOS_TR_STAMP_FIRST(p.trace, kTrProdFirstTma);
                    const uint32_t leader_bar = map_to_cta(smem_u32(&full[s]), 0);
                    mbar_arrive_expect_tx_cluster(leader_bar, tx_bytes);
                    tma_load_2d_pair(smem + S::kOffA + s * S::kABytes, &tmap_a, leader_bar, (int32_t)(kt * kGemmBlockK),
                                     (int32_t)m0);
                    if (p.b_kmajor) {  // the transposed copy [N, K]: this CTA's 128 columns are 128 rows of it
                        tma_load_2d_pair(smem + S::kOffB + s * S::kBBytes, &tmap_b, leader_bar, (int32_t)(kt * kGemmBlockK),
                                         (int32_t)n0);
                    } else {
                        tma_load_2d_pair(smem + S::kOffB + s * S::kBBytes, &tmap_b, leader_bar, (int32_t)n0,
                                         (int32_t)(kt * kGemmBlockK));
                    }
                    CATCCOS_TR_STAMP(p.trace, kTrProdLastTma);
                }
                alive = __all_sync(0xFFFFFFFFu, alive);
            }
        }
    } else if (warp == 5) {
        // ------------------------------- MMA issuer (leader CTA only) ---------------------
        // As in the single-CTA kernel the issuer issues the MMAs and the stage-releasing commit, nothing else.
        if (cta == 0 && lane == 0) {
            const bool bk = p.b_kmajor != 0u;
            const uint32_t idesc = make_idesc_mxf8(kPairBlockM, kPairBlockN, !bk) | ((p.a_fmt & 7u) << 7) |
                                   ((p.b_fmt & 7u) << 10);  // operand formats: E4M3 = 0, E5M2 = 1, E2M1 = 5
            const uint32_t my_tiles = (num_tiles > pair) ? (num_tiles - pair + num_pairs - 1) / num_pairs : 0u;
            const uint32_t total_it = my_tiles * k_tiles;

            const uint32_t hi_a = (uint32_t)(make_smem_desc(0, 16, 1024, 2) >> 32);
            const uint32_t hi_b = bk ? hi_a : (uint32_t)(make_smem_desc(0, 16384, 1024, 2) >> 32);
            const uint32_t a_lo0 = (uint32_t)make_smem_desc(0, 16, 1024, 2) | (smem_u32(smem + S::kOffA) >> 4);
            // each CTA holds 128 columns of B (one 128-byte swizzle row per K): MN-major
            const uint32_t b_lo0 = (uint32_t)make_smem_desc(0, bk ? 16 : 16384, 1024, 2) | (smem_u32(smem + S::kOffB) >> 4);
            const uint32_t kb_step_b = (bk ? 32u : 4096u) >> 4;
            const uint32_t sf_tmem0 = tmem_base + S::kSfCol;

            bool alive = true;
            auto stage_wait = [&](uint32_t s, uint32_t ph) {
                const unsigned long long t0 = CATCCOS_TR_NOW();
                (void)t0;
                alive = mbar_wait_cluster(&full[s], ph, p.status, 203, s, bar_ns);
                tcgen05_fence_after();
                CATCCOS_TR_ADD(p.trace, kTrMmaFullWaitNs, CATCCOS_TR_NOW() - t0);
            };
            auto issue_mma = [&](uint32_t a_lo, uint32_t b_lo, uint32_t sf, uint32_t kb, uint32_t d_col, uint32_t accumulate) {
                umma_mxf8_pair_lohi(d_col, a_lo + kb * (32u >> 4), hi_a, b_lo + kb * kb_step_b, hi_b,
                                    idesc_with_sf_id(idesc, kb), sf, sf + 4, accumulate);
            };

            if (total_it > 0) {
                stage_wait(0, 0);
            }
            uint32_t it = 0, s = 0, ph = 0;
            for (uint32_t ti = 0; alive && ti < my_tiles; ++ti) {
                const uint32_t acc = ti & 1u;
                const uint32_t acc_ph = (ti >> 1) & 1u;
                const uint32_t d_col = tmem_base + (acc ? S::kAccCol1 : 0u);
                const unsigned long long t0 = CATCCOS_TR_NOW();
                (void)t0;
                alive = mbar_wait_cluster(&tmem_empty[acc], acc_ph ^ 1u, p.status, 201, acc, bar_ns);
                if (ti > 0 && alive) {
                    alive = mbar_wait_cluster(&overlap_free[acc ^ 1u], ((ti - 1) >> 1) & 1u, p.status, 202, acc, bar_ns);
                }
                CATCCOS_TR_ADD(p.trace, kTrMmaAccWaitNs, CATCCOS_TR_NOW() - t0);
                tcgen05_fence_after();
                CATCCOS_TR_STAMP_FIRST(p.trace, kTrMmaFirst);
                for (uint32_t kt = 0; alive && kt < k_tiles; ++kt, ++it) {
                    const uint32_t a_lo = a_lo0 + s * (S::kABytes >> 4);
                    const uint32_t b_lo = b_lo0 + s * (S::kBBytes >> 4);
                    const uint32_t sf = sf_tmem0 + s * S::kSfSetCols;
                    const uint32_t s_next = (s + 1 == kStages) ? 0u : s + 1;
                    const uint32_t ph_next = ph ^ (s_next == 0u ? 1u : 0u);
                    const bool more = it + 1 < total_it;
                    issue_mma(a_lo, b_lo, sf, 0, d_col, kt != 0 ? 1u : 0u);
                    issue_mma(a_lo, b_lo, sf, 1, d_col, 1u);
                    issue_mma(a_lo, b_lo, sf, 2, d_col, 1u);
                    issue_mma(a_lo, b_lo, sf, 3, d_col, 1u);
                    tcgen05_commit_pair(&empty[s], 3);
                    if (more) {
                        stage_wait(s_next, ph_next);
                    }
                    s = s_next;
                    ph = ph_next;
                }
                tcgen05_commit_pair(&tmem_full[acc], 3);
                if (ti < kTraceTiles) {
                    CATCCOS_TR_STAMP(p.trace, kTrTileEnd + ti);
                }
                CATCCOS_TR_STAMP(p.trace, kTrMmaLast);
            }
        }
        __syncwarp();
    } else if (FUSED_QUANT && warp >= 10) {
        // ------------------------------- quantise-and-push producer -----------------------
        // Of the fourteen extra warps, eight quantise this rank's shard into the local stage (warps 10-19
        // except 13 and 17, which share a scheduler with the MMA issuer and must not compete with that
        // single thread for issue slots).  The other six (13, 17, 20-23) run the pusher, a copy loop that
        // issues an instruction only every few hundred cycles, and send finished items on to the peers.
        if (warp < 20u && (warp & 3u) != (5u & 3u)) {
            const uint32_t qw = warp - 10u - (warp > 13u ? 1u : 0u) - (warp > 17u ? 1u : 0u);  // 0..7
            quant_push_producer<true>(p.q, qw * 32u + lane, blockIdx.x, gridDim.x, 1);
        } else {
            const uint32_t pw = warp == 13u ? 0u : (warp == 17u ? 1u : warp - 18u);  // 0..5
            push_worker(p.push, lane, pw * gridDim.x + blockIdx.x, gridDim.x * kPushWarps, pw, gridDim.x, push_turn);
        }
    } else if (warp >= 6) {
        // ------------------------------- scale loaders (both CTAs) ------------------------
        // A scales of this CTA's 128 rows; B scales of all 256 columns of the pair's tile.
        constexpr uint32_t kNB = kPairBlockN / 32;
        const uint32_t j = warp - 6;
        if (p.flags == nullptr) {
            grid_dep_wait();  // the A scales are the output of the kernel launched just before (or: see the flags)
        }
        const uint32_t sf_row_bytes = p.K / 32;
        const uint32_t my_tiles = (num_tiles > pair) ? (num_tiles - pair + num_pairs - 1) / num_pairs : 0u;
        const uint32_t total_it = my_tiles * k_tiles;
        uint32_t cur_a[4], cur_lo[kNB], cur_hi[kNB];
        uint32_t nxt_a[4], nxt_lo[kNB], nxt_hi[kNB];
        uint32_t known_end = 0;  // K-tile iterations below this index have their rows in place
        bool alive = true;

        auto issue_loads = [&](uint32_t it, uint32_t (&ra)[4], uint32_t (&rlo)[kNB], uint32_t (&rhi)[kNB]) {
            const uint32_t seq = it / k_tiles;
            const uint32_t kt = it - seq * k_tiles;
            TileCoord tc = pair_tile_coord(pair + seq * num_pairs, n_tiles, m_tiles, p);
            const uint32_t m0 = tc.m_tile * kPairBlockM + cta * 128u;
            const uint32_t n0 = tc.n_tile * kPairBlockN;
            if (p.flags != nullptr && it >= known_end) {
                // this CTA's producer has usually seen these rows' flags already and said so in shared memory
                // one lane reads the word for the warp: the producer may be updating it, and the branch below holds
                // warp-wide operations, so every lane has to take the same side
                const uint32_t g = __shfl_sync(0xFFFFFFFFu, ld_acquire_cta_shared(gate), 0);
                if (g > it) {
                    known_end = g;
                } else {
                    const unsigned long long t0 = CATCCOS_TR_NOW();
                    (void)t0;
                    const uint32_t seg0 = kt / p.seg_ktiles;
                    const uint32_t nready = wait_rows_ready(p, m0, lane, seg0);
                    alive = alive && nready != 0u;
                    known_end = it + (min((seg0 + nready) * p.seg_ktiles, k_tiles) - kt);
                    if (lane == 0) {
                        CATCCOS_TR_ADD(p.trace, kTrSfGateWaitNs + j, CATCCOS_TR_NOW() - t0);
                    }
                }
            }
#pragma unroll
            for (uint32_t i = 0; i < 4; ++i) {
                const uint32_t row = m0 + i * 32 + lane;
                ra[i] = 0x7F7F7F7Fu;
                if (row < p.Mg) {
                    ra[i] = __ldcg(reinterpret_cast<const uint32_t*>(p.a_scales + (size_t)row * sf_row_bytes + kt * 4u));
                }
            }
#pragma unroll
            for (uint32_t i = 0; i < kNB; ++i) {
                const uint32_t n = n0 + i * 32 + lane;
                rlo[i] = 0x7F7Fu;
                rhi[i] = 0x7F7Fu;
                if (n < p.N) {
                    rlo[i] = __ldg(reinterpret_cast<const uint16_t*>(p.b_scales + ((size_t)(2 * kt) * p.N + n) * 2));
                    rhi[i] = __ldg(reinterpret_cast<const uint16_t*>(p.b_scales + ((size_t)(2 * kt + 1) * p.N + n) * 2));
                }
            }
        };

        uint32_t it = j;
        if (it < total_it) {
            issue_loads(it, cur_a, cur_lo, cur_hi);
        }
        for (; alive && it < total_it; it += kSfWarps) {
            const bool has_next = it + kSfWarps < total_it;
            if (has_next) {
                issue_loads(it + kSfWarps, nxt_a, nxt_lo, nxt_hi);
            }
            const uint32_t s = it % kStages;
            const uint32_t ph = (it / kStages) & 1u;
            const unsigned long long t1 = CATCCOS_TR_NOW();
            (void)t1;
            alive = mbar_wait_warp(&empty[s], ph ^ 1u, p.status, 205, s, bar_ns) && alive;
            if (lane == 0) {
                CATCCOS_TR_ADD(p.trace, kTrSfEmptyWaitNs + j, CATCCOS_TR_NOW() - t1);
            }
            uint8_t* sfa = smem + S::kOffSfa + s * S::kSfaBytes;
            uint8_t* sfb = smem + S::kOffSfb + s * S::kSfbBytes;
            *reinterpret_cast<uint4*>(sfa + lane * 16u) = make_uint4(cur_a[0], cur_a[1], cur_a[2], cur_a[3]);
#pragma unroll
            for (uint32_t h = 0; h < kNB / 4; ++h) {
                uint4 v;
                v.x = cur_lo[h * 4 + 0] | (cur_hi[h * 4 + 0] << 16);
                v.y = cur_lo[h * 4 + 1] | (cur_hi[h * 4 + 1] << 16);
                v.z = cur_lo[h * 4 + 2] | (cur_hi[h * 4 + 2] << 16);
                v.w = cur_lo[h * 4 + 3] | (cur_hi[h * 4 + 3] << 16);
                *reinterpret_cast<uint4*>(sfb + h * 512u + lane * 16u) = v;
            }
            fence_proxy_async_shared();
            __syncwarp();
            if (lane == 0) {
                // Both CTAs report their atoms to the leader; the leader's scale loader then copies both CTAs'
                // atoms into both CTAs' tensor memory (one cta_group::2 copy does the same offsets in the two) and
                // its commit is the third arrival on the leader's full barrier.  The MMA issuer copies nothing:
                // a thread gets a tcgen05 instruction out only every ~70 cycles.
                mbar_arrive_cluster(map_to_cta(smem_u32(&atoms_written[s]), 0));
                if (cta == 0) {
                    mbar_wait_cluster(&atoms_written[s], ph, p.status, 207, s, bar_ns);
                    tcgen05_fence_after();
                    const uint32_t hi_sf = (uint32_t)(make_smem_desc(0, 0, 128, 0) >> 32);
                    const uint32_t sf_t = tmem_base + S::kSfCol + s * S::kSfSetCols;
                    tcgen05_cp_sf_pair_lohi(sf_t, smem_u32(sfa) >> 4, hi_sf);
                    tcgen05_cp_sf_pair_lohi(sf_t + 4, smem_u32(sfb) >> 4, hi_sf);
                    tcgen05_cp_sf_pair_lohi(sf_t + 8, (smem_u32(sfb) >> 4) + (512u >> 4), hi_sf);
                    tcgen05_commit_pair(&full[s], 1);
                }
            }
            if (has_next) {
#pragma unroll
                for (uint32_t i = 0; i < 4; ++i) cur_a[i] = nxt_a[i];
#pragma unroll
                for (uint32_t i = 0; i < kNB; ++i) {
                    cur_lo[i] = nxt_lo[i];
                    cur_hi[i] = nxt_hi[i];
                }
            }
        }
    } else {
        // ------------------------------- epilogue (both CTAs, own 128 rows) ---------------
        const uint32_t q = warp;
        OutT* c = reinterpret_cast<OutT*>(p.c);
        constexpr uint32_t kChunks = kPairBlockN / 32;
        uint32_t ti = 0;
        for (uint32_t tile = pair; tile < num_tiles; tile += num_pairs, ++ti) {
            TileCoord tc = pair_tile_coord(tile, n_tiles, m_tiles, p);
            const uint32_t m0 = tc.m_tile * kPairBlockM + cta * 128u;
            const uint32_t n0 = tc.n_tile * kPairBlockN;
            const uint32_t acc = ti & 1u;
            const uint32_t acc_ph = (ti >> 1) & 1u;
            const uint32_t d_col = acc ? S::kAccCol1 : 0u;
            const unsigned long long t0 = CATCCOS_TR_NOW();
            (void)t0;
            const bool alive = mbar_wait_warp(&tmem_full[acc], acc_ph, p.status, 206, acc, bar_ns);
            if (q == 0 && lane == 0) {
                CATCCOS_TR_ADD(p.trace, kTrEpiWaitNs, CATCCOS_TR_NOW() - t0);
            }
            if (!alive) {
                break;  // an accumulator that never filled is not written out
            }
            tcgen05_fence_after();
            const uint32_t row = m0 + q * 32 + lane;
            for (uint32_t ci = 0; ci < kChunks; ++ci) {
                uint32_t chunk = ci;
                if (acc == 0) {  // the shared columns first
                    chunk = ci < S::kOverlapChunks ? kChunks - S::kOverlapChunks + ci : ci - S::kOverlapChunks;
                }
                uint32_t r[32];
                tmem_ld_32x32(tmem_base + ((q * 32u) << 16) + d_col + chunk * 32u, r);
                tmem_ld_wait();
                if (ci == S::kOverlapChunks - 1) {
                    tcgen05_fence_before();
                    __syncwarp();
                    if (lane == 0) {
                        mbar_arrive_cluster(map_to_cta(smem_u32(&overlap_free[acc]), 0));
                    }
                }
                store_c_chunk<OutT>(c, p, row, n0 + chunk * 32u, r);
            }
            publish_tile_rows<OutT>(p, m0 + q * 32u, tc.n_tile, n_tiles, lane);
            tcgen05_fence_before();
            __syncwarp();
            if (lane == 0) {
                mbar_arrive_cluster(map_to_cta(smem_u32(&tmem_empty[acc]), 0));
                if (q == 0) {
                    CATCCOS_TR_STAMP(p.trace, kTrEpiLast);
                }
            }
        }
    }

    tcgen05_fence_before();
    __syncthreads();
    drain_after_abort(p.status);  // both CTAs stay while loads that report to the other's barriers may be in flight
    cluster_sync_all();  // nobody leaves while the other CTA may still arrive on its barriers
    if (threadIdx.x == 0) {
        CATCCOS_TR_STAMP(p.trace, kTrCtaEnd);
    }
    if (warp == 5) {
        tcgen05_fence_after();
        tmem_dealloc_pair(tmem_base, kTmemCols);
    }
}

}  // namespace catccos
