// dQ kernel. Replaces `_bwd_q_kernel` (flash_triton.py:323-431): per block of 128 queries,
// walk the visited key tiles, recompute P = exp2(S*scale*log2e - LSE), dP = dO V^T,
// dS = P * (dP - delta) with masked entries zeroed, dQ += dS K, and scale by sm_scale at the end.
//
// One CTA = one query block of one (batch, head), 12 warps:
//   warps 0-7  two compute groups; thread r of group g owns query row r and key columns
//              [64g, 64g+64) of every tile
//   warp 8     TMA producer (Q and dO once, K ring, V ring)
//   warps 9,10 tcgen05.mma issuers (warp 9 also owns the TMEM allocation)
// TMEM columns: S0 [0,128) S1 [128,256) dP [256,384) dQ [384,384+D). dS (input dtype) is
// written over the first half of each group's own S columns and fed to the dQ MMA from TMEM.
#include "common.cuh"
#include "params.cuh"
#include "trace.cuh"

namespace fa {

template <int D>
struct DqSmem {
    static constexpr int NSK = (D == 128) ? 3 : 4;
    static constexpr int NSV = (D == 128) ? 2 : 4;
    static constexpr int TILE = kBlk * D * 2;
    static constexpr int BOX = kBlk * 64 * 2;
    static constexpr int NBOX = D / 64;
    static constexpr int off_q = 0;
    static constexpr int off_do = TILE;
    static constexpr int off_k = 2 * TILE;
    static constexpr int off_v = off_k + NSK * TILE;
    static constexpr int off_list = off_v + NSV * TILE;
    static constexpr int off_bar = off_list + kListCap * 2;
    // qdo_full, k_full[NSK], v_full[NSV], k_empty[NSK], v_empty[NSV], s_full[2], ds_full[2], dp_full, done
    static constexpr int n_bar = 1 + 2 * NSK + 2 * NSV + 6;
    static constexpr int off_misc = off_bar + n_bar * 8;
    static constexpr int total = off_misc + 16;
};

template <int D, bool BF16>
__global__ void __launch_bounds__(kAttnThreads, 1)
bwd_dq_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
              const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmdO,
              const __grid_constant__ CUtensorMap tmdQ, const DqParams p) {
    using S = DqSmem<D>;
    constexpr int NSK = S::NSK, NSV = S::NSV;
    extern __shared__ __align__(1024) uint8_t smem[];
    const uint32_t sbase = smem_u32(smem);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    FA_TRACE_DECL

    const MaskArgs& mk = p.mask;
    const int qb = mk.L.nQ - 1 - int(blockIdx.x);
    const int h = blockIdx.y, b = blockIdx.z;
    const int hk = h / p.G;
    const int he = (mk.He == 1) ? 0 : h;

    uint16_t* list = reinterpret_cast<uint16_t*>(smem + S::off_list);
    volatile int* misc = reinterpret_cast<volatile int*>(smem + S::off_misc);
    const uint32_t bar0 = sbase + S::off_bar;
    auto BAR = [&](int i) { return bar0 + 8u * uint32_t(i); };
    const int B_QDO = 0, B_KFULL = 1, B_VFULL = B_KFULL + NSK, B_KEMPTY = B_VFULL + NSV, B_VEMPTY = B_KEMPTY + NSK,
              B_SFULL = B_VEMPTY + NSV, B_DSFULL = B_SFULL + 2, B_DPFULL = B_DSFULL + 2, B_DONE = B_DPFULL + 1;
    Abort ab{misc + 1, p.status};

    const uint32_t sQ = sbase + S::off_q, sdO = sbase + S::off_do;
    auto sK = [&](int s) { return sbase + S::off_k + uint32_t(s) * S::TILE; };
    auto sV = [&](int s) { return sbase + S::off_v + uint32_t(s) * S::TILE; };

    // The producer thread sets up the barriers itself, so that it can start the Q / dO loads (which
    // do not depend on the plan) before anything else happens in the CTA.
    const bool producer = (warp == 8 && lane == 0);
    if (producer) {
        mbar_init(BAR(B_QDO), 1);
        for (int s = 0; s < NSK; ++s) { mbar_init(BAR(B_KFULL + s), 1); mbar_init(BAR(B_KEMPTY + s), 1); }
        for (int s = 0; s < NSV; ++s) { mbar_init(BAR(B_VFULL + s), 1); mbar_init(BAR(B_VEMPTY + s), 1); }
        for (int w = 0; w < 2; ++w) { mbar_init(BAR(B_SFULL + w), 1); mbar_init(BAR(B_DSFULL + w), 256); }
        mbar_init(BAR(B_DPFULL), 1);
        mbar_init(BAR(B_DONE), 1);
        misc[1] = (*reinterpret_cast<volatile int*>(p.status) != 0 || (sbase & 1023u) != 0) ? 1 : 0;
        misc[2] = 0;
        fence_mbar_init();
        if (misc[1] == 0) {
            tma_prefetch_desc(&tmQ); tma_prefetch_desc(&tmdO); tma_prefetch_desc(&tmK); tma_prefetch_desc(&tmV);
            mbar_expect_tx(BAR(B_QDO), 2 * S::TILE);
            for (int x = 0; x < S::NBOX; ++x) {
                tma_load_4d(sQ + x * S::BOX, &tmQ, BAR(B_QDO), x * 64, qb * kBlk, h, b);
                tma_load_4d(sdO + x * S::BOX, &tmdO, BAR(B_QDO), x * 64, qb * kBlk, h, b);
            }
        }
    }
    if (warp == 9) {
        tmem_alloc(sbase + S::off_misc, 512);
        tmem_relinquish();
    }
    int lo, hi;
    kv_range(mk, b, he, qb, lo, hi);
    int n = hi - lo;
    if (n > kListCap) n = kListCap;
    // ... and the first visited key block's K and V as soon as it knows which block that is
    // (normally candidate 0: the range starts at a visited block)
    if (producer && misc[1] == 0) {
        int c0 = 0;
        while (c0 < n && !(classify_from_plan(mk, b, he, qb, lo + c0) & TILE_VISIT)) ++c0;
        if (c0 < n) {
            mbar_expect_tx(BAR(B_KFULL + 0), S::TILE);
            mbar_expect_tx(BAR(B_VFULL + 0), S::TILE);
            for (int x = 0; x < S::NBOX; ++x) {
                tma_load_4d(sK(0) + x * S::BOX, &tmK, BAR(B_KFULL + 0), x * 64, (lo + c0) * kBlk, hk, b);
                tma_load_4d(sV(0) + x * S::BOX, &tmV, BAR(B_VFULL + 0), x * 64, (lo + c0) * kBlk, hk, b);
            }
        }
    }
    for (int i = tid; i < n; i += kAttnThreads) list[i] = uint16_t(classify_from_plan(mk, b, he, qb, lo + i));
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    if (warp == 0) {
        const int Tn = compact_visit_list(list, n, lane);
        if (lane == 0) misc[2] = Tn;
    }
    __syncthreads();
    const uint32_t tmem = uint32_t(misc[0]);
    const int T = misc[2];
    const bool aborted = misc[1] != 0;

    if (warp >= 8) {
        setmaxnreg_dec<56>();
        if (aborted || T == 0) {
        } else if (warp == 8) {
            // ------------------------------ TMA producer ------------------------------
            if (lane == 0) {
                bool ok = true;
                for (int t = 0; t <= T && ok; ++t) {  // K runs one tile ahead of V; K(0), V(0) are already under way
                    if (t < T && t > 0) {
                        const int kb = lo + (list[t] & 1023);
                        const int st = t % NSK, use = t / NSK;
                        if (use > 0) ok = mbar_wait(BAR(B_KEMPTY + st), (use - 1) & 1, ab, ST_WAIT_TIMEOUT + 21);
                        if (!ok) break;
                        mbar_expect_tx(BAR(B_KFULL + st), S::TILE);
                        for (int x = 0; x < S::NBOX; ++x)
                            tma_load_4d(sK(st) + x * S::BOX, &tmK, BAR(B_KFULL + st), x * 64, kb * kBlk, hk, b);
                    }
                    if (t >= 2) {
                        const int tv = t - 1;
                        const int kb = lo + (list[tv] & 1023);
                        const int st = tv % NSV, use = tv / NSV;
                        if (use > 0) ok = mbar_wait(BAR(B_VEMPTY + st), (use - 1) & 1, ab, ST_WAIT_TIMEOUT + 22);
                        if (!ok) break;
                        mbar_expect_tx(BAR(B_VFULL + st), S::TILE);
                        for (int x = 0; x < S::NBOX; ++x)
                            tma_load_4d(sV(st) + x * S::BOX, &tmV, BAR(B_VFULL + st), x * 64, kb * kBlk, hk, b);
                    }
                }
            }
        } else if (warp == 9 || warp == 10) {
            // ------------------------------ MMA issuers ------------------------------
            // Two issuing threads, so that the blocking tcgen05.mma issue and barrier round trips of
            // one stream do not delay the other:
            //   warp 9 : S(0), S(1); then per tile dQ(t) += dS K(t) followed by S(t+2) (which
            //            overwrites dS(t): same thread, in order)
            //   warp 10: dP(t+1) = dO V(t+1)^T as soon as dS(t) has been written (dP columns free)
            if (lane == 0) {
                constexpr uint32_t idesc_s = make_idesc(BF16, 128, 128, false, false);
                constexpr uint32_t idesc_dq = make_idesc(BF16, 128, D, false, true);
                constexpr uint64_t desc_mn = desc_mn_major(S::BOX);
                bool ok = mbar_wait(BAR(B_QDO), 0, ab, ST_WAIT_TIMEOUT + 23);
                auto k_ready = [&](int t) { return mbar_wait(BAR(B_KFULL + t % NSK), (t / NSK) & 1, ab, ST_WAIT_TIMEOUT + 24); };
                auto v_ready = [&](int t) { return mbar_wait(BAR(B_VFULL + t % NSV), (t / NSV) & 1, ab, ST_WAIT_TIMEOUT + 25); };
                auto ss_mmas = [&](uint32_t d, uint32_t a_tile, uint32_t b_tile) {
#pragma unroll
                    for (int kk = 0; kk < D / 16; ++kk) {
                        const uint32_t off = uint32_t(kk >> 2) * S::BOX + uint32_t(kk & 3) * 32u;
                        umma_ss(d, smem_desc_at(kDescKMajor, a_tile + off), smem_desc_at(kDescKMajor, b_tile + off),
                                idesc_s, kk > 0);
                    }
                };
                if (warp == 9) {
                    for (int t = 0; t < 2 && t < T && ok; ++t) {
                        ok = k_ready(t);
                        if (ok) {
                            tc_fence_after();
                            ss_mmas(tmem + uint32_t(t) * 128u, sQ, sK(t % NSK));
                            umma_commit(BAR(B_SFULL + t));
                        }
                    }
                    for (int t = 0; t < T && ok; ++t) {
                        const int st = t % NSK;
                        FA_TRACE_EV(2, 3);
                        ok = mbar_wait(BAR(B_DSFULL + (t & 1)), (t >> 1) & 1, ab, ST_WAIT_TIMEOUT + 26);
                        if (!ok) break;
                        tc_fence_after();
                        FA_TRACE_EV(2, 4);
                        const uint32_t a = tmem + uint32_t(t & 1) * 128u;
#pragma unroll
                        for (int kk = 0; kk < kBlk / 16; ++kk) {
                            const uint32_t acol = (kk < 4) ? uint32_t(kk) * 8u : 64u + uint32_t(kk - 4) * 8u;
                            umma_ts(tmem + 384u, a + acol, smem_desc_at(desc_mn, sK(st) + uint32_t(kk) * 2048u), idesc_dq,
                                    (t > 0 || kk > 0) ? 1u : 0u);
                        }
                        umma_commit(BAR(B_KEMPTY + st));
                        // K(t+2) reuses the stage that dQ(t-1) releases, so it is waited for only now
                        if (t + 2 < T) {
                            ok = k_ready(t + 2);
                            if (ok) {
                                tc_fence_after();
                                ss_mmas(a, sQ, sK((t + 2) % NSK));
                                umma_commit(BAR(B_SFULL + (t & 1)));
                            }
                        }
                        FA_TRACE_EV(2, 5);
                    }
                    if (ok) umma_commit(BAR(B_DONE));
                } else {
                    for (int t = 0; t < T && ok; ++t) {
                        const int st = t % NSV;
                        ok = v_ready(t);
                        // dP(t) may overwrite the dP columns once every thread has read dP(t-1)
                        if (ok && t > 0) ok = mbar_wait(BAR(B_DSFULL + ((t - 1) & 1)), ((t - 1) >> 1) & 1, ab, ST_WAIT_TIMEOUT + 26);
                        if (!ok) break;
                        tc_fence_after();
                        ss_mmas(tmem + 256u, sdO, sV(st));
                        umma_commit(BAR(B_VEMPTY + st));
                        umma_commit(BAR(B_DPFULL));
                    }
                }
            }
        }
        __syncwarp();
    } else {
        setmaxnreg_inc<224>();
        // ------------------------------ compute groups ------------------------------
        const int w = warp >> 2;
        const int r = tid & 127;
        const uint32_t lane_base = uint32_t((warp & 3) * 32) << 16;
        const int row = qb * kBlk + r;
        const int cbase = 64 * w;
        const float c = p.scale_log2;
        const int64_t bh_ids = int64_t(b) * mk.He + he;
        const int64_t bh_row = (int64_t(b) * p.H + h) * mk.L.Mpad + row;
        const int qc = (mk.mode == 1) ? mk.plan[mk.L.off_qc + bh_ids * mk.L.Mpad + row] : 0;
        const float lse = p.lse[bh_row];
        const float delta = p.delta[bh_row];
        bool ok = !aborted;

        for (int t = 0; t < T && ok; ++t) {
            const uint32_t entry = list[t];
            const uint32_t fl = entry >> 10;
            const int k0 = (lo + int(entry & 1023u)) * kBlk + cbase;  // first key column of this thread
            const uint32_t tS = tmem + lane_base + uint32_t(t & 1) * 128u + uint32_t(cbase);
            if (r == 0) FA_TRACE_EV(w, 10);
            ok = mbar_wait(BAR(B_SFULL + (t & 1)), (t >> 1) & 1, ab, ST_WAIT_TIMEOUT + 27);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tc_fence_after();
            uint32_t sr[64];
            tmem_ld32(tS, sr);
            tmem_ld32(tS + 32u, sr + 32);
            tc_wait_ld();
            float* pr = reinterpret_cast<float*>(sr);
            if (r == 0) FA_TRACE_EV(w, 12);
            {
                // P = exp2(S*c - LSE) on packed pairs
                const uint64_t c2 = pack_f2(c, c), nl2 = pack_f2(-lse, -lse);
#pragma unroll
                for (int j = 0; j < 32; ++j) {
                    float x0, x1;
                    unpack_f2(fma_f2(pack_f2(pr[2 * j], pr[2 * j + 1]), c2, nl2), x0, x1);
                    pr[2 * j] = fast_exp2(x0);
                    pr[2 * j + 1] = fast_exp2(x1);
                }
            }
            if (fl & (TILE_BOUND | TILE_DOC)) {
                int lim = 63;
                if (fl & TILE_BOUND) {
                    int jmax = mk.N - 1;
                    if (mk.causal) jmax = min(jmax, row + mk.gap);
                    lim = jmax - k0;
                }
                if ((fl & TILE_DOC) && qc < 0) {
                    const int4* kc4 = reinterpret_cast<const int4*>(mk.plan + mk.L.off_kc + bh_ids * mk.L.Npad + k0);
#pragma unroll
                    for (int q = 0; q < 16; ++q) {
                        const int4 kc = __ldg(kc4 + q);
                        pr[4 * q + 0] = (kc.x == qc && 4 * q + 0 <= lim) ? pr[4 * q + 0] : 0.f;
                        pr[4 * q + 1] = (kc.y == qc && 4 * q + 1 <= lim) ? pr[4 * q + 1] : 0.f;
                        pr[4 * q + 2] = (kc.z == qc && 4 * q + 2 <= lim) ? pr[4 * q + 2] : 0.f;
                        pr[4 * q + 3] = (kc.w == qc && 4 * q + 3 <= lim) ? pr[4 * q + 3] : 0.f;
                    }
                } else {
#pragma unroll
                    for (int j = 0; j < 64; ++j) pr[j] = (j <= lim) ? pr[j] : 0.f;
                }
            }
            if (r == 0) FA_TRACE_EV(w, 13);
            ok = mbar_wait(BAR(B_DPFULL), t & 1, ab, ST_WAIT_TIMEOUT + 28);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tc_fence_after();
            if (r == 0) FA_TRACE_EV(w, 16);
            uint32_t pk[32];
#pragma unroll
            for (int q = 0; q < 2; ++q) {
                uint32_t dp[32];
                tmem_ld32(tmem + lane_base + 256u + uint32_t(cbase) + uint32_t(q) * 32u, dp);
                tc_wait_ld();
                // masked entries have P == 0 exactly and dP - delta is finite, so dS is 0 there
                // (flash_triton.py:400-414)
                const uint64_t nd2 = pack_f2(-delta, -delta);
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    float d0, d1;
                    unpack_f2(mul_f2(pack_f2(pr[32 * q + 2 * j], pr[32 * q + 2 * j + 1]),
                                     add_f2(pack_f2(__uint_as_float(dp[2 * j]), __uint_as_float(dp[2 * j + 1])), nd2)),
                              d0, d1);
                    pk[16 * q + j] = pack2<BF16>(d0, d1);
                }
            }
            tmem_st32(tS, pk);
            tc_wait_st();
            tc_fence_before();
            mbar_arrive(BAR(B_DSFULL + (t & 1)));
            if (r == 0) FA_TRACE_EV(w, 17);
        }

        // ------------------------------ epilogue ------------------------------
        if (ok && T > 0) ok = mbar_wait(BAR(B_DONE), 0, ab, ST_WAIT_TIMEOUT + 29);
        // without visited tiles nobody has waited for the Q / dO loads yet, and Q's tile is the staging area
        if (ok && T == 0) ok = mbar_wait(BAR(B_QDO), 0, ab, ST_WAIT_TIMEOUT + 30);
        ok = __all_sync(0xffffffffu, ok);
        tc_fence_after();
        const bool healthy = ok && misc[1] == 0;
        {
            // dQ * sm_scale (flash_triton.py:425) goes out through shared memory: each thread writes
            // its half row into the (now dead) Q tile in the tensor map's 128-byte-swizzled layout,
            // then one thread issues the TMA store, which clips rows >= M.
            constexpr int HALF = D / 2;
            const uint32_t c0 = uint32_t(w) * HALF;
            uint8_t* stage = smem + S::off_q;
#pragma unroll
            for (int q = 0; q < HALF / 32; ++q) {
                uint32_t x[32];
                tmem_ld32(tmem + lane_base + 384u + c0 + uint32_t(q) * 32u, x);
                tc_wait_ld();
                uint32_t out[16];
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    const float v0 = (T > 0) ? __uint_as_float(x[2 * j]) * p.sm_scale : 0.f;
                    const float v1 = (T > 0) ? __uint_as_float(x[2 * j + 1]) * p.sm_scale : 0.f;
                    out[j] = pack2<BF16>(v0, v1);
                }
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int cg = int(c0) / 8 + 4 * q + i;  // 16-byte chunk of the row
                    const int box = cg >> 3, ch = cg & 7;
                    uint4* dst = reinterpret_cast<uint4*>(stage + box * S::BOX + r * 128 + ((ch ^ (r & 7)) << 4));
                    *dst = make_uint4(out[4 * i], out[4 * i + 1], out[4 * i + 2], out[4 * i + 3]);
                }
            }
            fence_proxy_async();
            named_bar_sync(1, 256);
            if (tid == 0 && healthy) {
                for (int x = 0; x < S::NBOX; ++x) tma_store_4d(&tmdQ, sbase + S::off_q + x * S::BOX, x * 64, qb * kBlk, h, b);
                tma_store_commit();
                tma_store_wait_read();
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 9) {
        tc_fence_after();
        tmem_dealloc(tmem, 512);
    }
}

template <int D, bool BF16>
static cudaError_t launch_dq_t(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv,
                               const CUtensorMap& tdo, const CUtensorMap& tdq, const DqParams& p, int B,
                               cudaStream_t stream) {
    auto kern = bwd_dq_kernel<D, BF16>;
    constexpr int smem = DqSmem<D>::total;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return e;
    dim3 grid(p.mask.L.nQ, p.H, B);
    kern<<<grid, kAttnThreads, smem, stream>>>(tq, tk, tv, tdo, tdq, p);
    return cudaGetLastError();
}

FA_TRACE_DUMP_FN(fa_trace_dump_dq)

cudaError_t launch_bwd_dq(int D, bool bf16, const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv,
                          const CUtensorMap& tdo, const CUtensorMap& tdq, const DqParams& p, int B, cudaStream_t stream) {
    if (D == 128) return bf16 ? launch_dq_t<128, true>(tq, tk, tv, tdo, tdq, p, B, stream)
                              : launch_dq_t<128, false>(tq, tk, tv, tdo, tdq, p, B, stream);
    return bf16 ? launch_dq_t<64, true>(tq, tk, tv, tdo, tdq, p, B, stream)
                : launch_dq_t<64, false>(tq, tk, tv, tdo, tdq, p, B, stream);
}

}  // namespace fa
