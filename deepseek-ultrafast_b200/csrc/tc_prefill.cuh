// tcgen05 GEMM for prefill-size token tiles: 128 tokens x TWO 128-row weight tiles per CTA step.  Grouped MXFP4
// expert GEMMs (gate/up + SwiGLU, down) and the dense FP8 projection; MX (power-of-two, applied by the tensor core)
// or DS (fp32 per 1x128, promoted per K tile) activation scales.
//
// Measured on B200 with the decode kernel (tc_stream.cuh) at 128-token tiles: a tcgen05.mma occupies its issuing
// thread for about as long as it occupies the tensor pipe (97 cycles at N = 128), and everything else that thread
// does per tile (the wait on the stage, fences, scale copies, the commit: ~350 cycles) is added serially, so one
// issuer keeps the pipe barely half busy; the ring of six 33 KB stages also covers too little latency.  Here
//   * a stage holds one activation tile (128 tokens x 128 K) and the tiles of two adjacent weight row tiles, so
//     every activation byte brought into shared memory feeds 256 weight rows (a third less ingest per flop);
//   * two issuer warps each own one of the two row tiles: the bookkeeping of one overlaps the MMAs of the other, and
//     the summation order of every output is fixed (results do not depend on timing);
//   * sixteen epilogue warps drain an accumulator into registers (64 columns per thread), release the tensor
//     memory, and run the SwiGLU / store epilogue while the next item's MMAs proceed;
//   * work items are dealt so that the items in flight share weight tiles and token tiles through L2 (see the item
//     order in the kernel): every input byte comes from HBM once.
// Replaces tc_moe_w13 / tc_moe_w2 (crates/kernels/cu/tcmoe.cu:184-588) and tc_gemm_fp8 / tc_gemm_fp8p
// (cu/tcgemm.cu:20-288); the weights come straight from the tile records (no in-kernel re-layout warps,
// cu/tcmoe.cu:412-456).
#pragma once
#include "tc_stream.cuh"

namespace dsuf {

constexpr int KID_TCP = 4;


// NTOK: token rows per step.  128 is the plan's slot.  64 walks every slot as two halves: a thread of the epilogue
// then holds 32 instead of 64 accumulators, so a whole tile's columns fit in flight in one tensor-memory load, and the
// smaller stage leaves room for a fifth one.  Used where it measured faster: the dense GEMM with DS (fp32) scales.
template <int NTOK>
struct TcpCfgT {
    static constexpr int A_BYTES = 16384;            // one weight tile, FP4 widened to 8-bit containers by TMA
    static constexpr int B_OFF = 2 * A_BYTES;        // NTOK token rows of 128 bytes
    static constexpr int SFA_OFF = B_OFF + NTOK * 128;  // two weight scale atoms (512 bytes each)
    static constexpr int SFB_OFF = SFA_OFF + 1024;   // activation scale atom
    static constexpr int STAGE = SFB_OFF + 1024;     // 51200 / 43008: multiples of 1024
    static constexpr int STAGES = NTOK == 128 ? 4 : 5;
    static constexpr int ONES_OFF = STAGE * STAGES;  // 512-byte atom of UE8M0 1.0 (DS activations)
    static constexpr int SMEM = STAGE * STAGES + 512 + 1024;
    static constexpr int EPI_WARP0 = 4;              // warps 4..19: four groups of four (accumulator x column half)
    static constexpr int THREADS = (EPI_WARP0 + 16) * 32;
    static constexpr int TM_SFA = 384, TM_SFB = 448, TM_COLS = 512;  // accumulators: columns 0..383
};
using TcpCfg = TcpCfgT<128>;

// warp 0 / 2: producers (weight row tile 0 + activation tile / weight row tile 1 + activation scales),
// 1 / 3: MMA issuers (accumulator 0 / 1), 4..19: epilogue (640 threads: 96 registers each)
// AMX = 1: UE8M0 activation scales per 1x32, applied by the tensor core; the whole K accumulates in tensor memory.
// AMX = 0: fp32 activation scales per 1x128 (DS geometry): every 128-K tile is promoted into fp32 registers with
//          its scales.  The two issuers rotate over three accumulators, so one is read out while two take MMAs.
// FMT / WMX: FP4 expert tiles (UE8M0 weight scales in the tile record) or dense FP8 weights with UE8M0 (MX) or fp32
// 128x128 (DS) scales.  EPI_DENSE: the "slots" are the 128-row tiles of the a.m token rows of one dense matrix.
template <int EPI, int AMX, int FMT = FMT_FP4, int WMX = 1, int NTOK = 128>
__global__ void __launch_bounds__(TcpCfgT<NTOK>::THREADS, 1) tc_prefill_kernel(const __grid_constant__ StreamArgs a) {
    using Cfg = TcpCfgT<NTOK>;
    static_assert(WMX || !AMX, "fp32 weight scales are promoted per K tile together with fp32 activation scales");
    static_assert(NTOK == 128 || NTOK == 64, "token rows per step");
    constexpr int HALVES = 128 / NTOK;  // steps a 128-row slot is walked in
    constexpr int CPT = NTOK / 2;       // token columns per epilogue thread
    // (expert, first token row, token rows (<= 0: nothing to do), -) of sub-slot vs = slot * HALVES + half
    auto slot_of = [&](int vs) -> int4 {
        const int slot = vs / HALVES, r0 = (vs % HALVES) * NTOK;
        if (EPI == EPI_DENSE) return make_int4(0, slot * 128 + r0, min(NTOK, a.m - slot * 128 - r0), 0);
        const int4 sl = a.slots[slot];
        return make_int4(sl.x, sl.y + r0, min(NTOK, sl.z - r0), 0);
    };
    constexpr int S = Cfg::STAGES;
    constexpr int XR = 8;  // ring of fp32 activation scales (DS): outlives the stage, read after the MMAs completed
    __shared__ __align__(16) float s_xs[AMX ? 4 : XR * NTOK];
    extern __shared__ uint8_t smem_raw[];
    uint8_t* ring = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    __shared__ __align__(8) uint64_t full_bar[S], empty_bar[S], tfull_bar[6], tempty_bar[6];  // [accumulator][issuer]
    __shared__ uint32_t s_tmem;
    __shared__ int s_efirst[EPI == EPI_DENSE ? 1 : 512], s_elast[EPI == EPI_DENSE ? 1 : 512];  // slot range of every expert

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int G = gridDim.x, c = blockIdx.x;
    // row-tile pairs per expert; with an odd number of row tiles the last pair's second half streams the last tile once
    // more (its outputs are dropped): one step in RT of the weight bytes read twice instead of a second kernel
    const int RT = a.RT, KT = a.KT, RP = (RT + 1) >> 1;
    bool dead = false;  // set by the first expired wait: nothing is waited for again, the loops stay finite

    if (warp == 1) {
        tmem_alloc(&s_tmem, Cfg::TM_COLS);
        tmem_relinquish();
    }
    if (tid == 0) {
        for (int s = 0; s < S; ++s) {
            mbar_init(&full_bar[s], 2 + 32);  // one expect_tx per producer warp + 32 cp.async lanes
            mbar_init(&empty_bar[s], 2);      // one tcgen05.commit per issuer
        }
        for (int j = 0; j < 6; ++j) {
            mbar_init(&tfull_bar[j], 1);
            mbar_init(&tempty_bar[j], 8);     // the eight epilogue warps of the accumulator
        }
        mbar_fence_init();
    }
    if (!AMX && tid >= 64 && tid < 192) ((uint32_t*)(ring + Cfg::ONES_OFF))[tid - 64] = 0x7f7f7f7fu;  // one atom of UE8M0 1.0
    fence_proxy_async();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tm = s_tmem;
    pdl_wait();
    pdl_launch_dependents();  // dependents still wait for this grid to finish; only their prologues overlap

    // Items = (slot, row-tile pair), dealt to the CTAs round-robin in the order [expert][group of <= 32 slots][row-tile
    // pair][slot of the group]: the G items in flight at any time are a block of a few row-tile pairs x the slots of one
    // group, so a weight tile is fetched from HBM once per group (not once per slot) and a group's token tiles stay in L2
    // while its row-tile pairs go by.  (Dealing contiguous (slot, pair) ranges instead read 13 x the unique bytes from
    // HBM on a 2048-token profile and made the kernel HBM-bound.)
    const int nslots = EPI == EPI_DENSE ? (a.m + 127) / 128 : *a.nslots;
    const int nitems = nslots * HALVES * RP;  // far below 2^31: slots <= permuted rows / 128 + experts
    constexpr int SG = 32;
    if (EPI != EPI_DENSE) {
        // first and last slot of every expert (slots are sorted by expert)
        for (int sidx = tid; sidx < nslots; sidx += Cfg::THREADS) {
            const int e = a.slots[sidx].x;
            if (sidx == 0 || a.slots[sidx - 1].x != e) s_efirst[e] = sidx;
            if (sidx == nslots - 1 || a.slots[sidx + 1].x != e) s_elast[e] = sidx;
        }
        __syncthreads();
    }
    auto item_of = [&](int i, int& slot, int& rp) {
        int f = 0, n = nslots * HALVES;  // in sub-slots
        if (EPI != EPI_DENSE) {
            const int e = a.slots[i / (RP * HALVES)].x;  // item blocks of an expert start at multiples of RP * HALVES
            f = s_efirst[e] * HALVES;
            n = (s_elast[e] + 1) * HALVES - f;
        }
        const int l = i - f * RP;
        const int grp = l / (SG * RP), lg = l - grp * (SG * RP);
        const int ng = min(SG, n - grp * SG);
        rp = lg / ng;
        slot = f + grp * SG + (lg - rp * ng);
    };
    const int ibeg = c, iend = nitems;  // it = c, c + G, ...

    if (warp == 0 || warp == 2) {
        // ================= producers =================
        // warp 0: weight row tile 2*rp (codes + scale atom) and the activation tile;
        // warp 2: weight row tile 2*rp + 1 and the activation scales (4-byte async copies into the scale atom)
        const int j = warp >> 1;
        if (ibeg < iend) {
            if (lane == 0) { prefetch_tmap(&a.tm_w); prefetch_tmap(&a.tm_x); }
            const uint64_t pol = policy_evict_last();  // scale atoms and token rows; the weight tiles take the default policy
            int s = 0;
            uint32_t ph = 0;
            int n = 0;
            for (int it = ibeg; it < iend; it += G) {
                int slot, rp;
                item_of(it, slot, rp);
                const int4 sl = slot_of(slot);
                if (sl.z <= 0) continue;  // second half of a slot with at most NTOK rows: every role skips it
                const int xrow0 = sl.y;
                int tile = (int)((((long long)sl.x * RT) + min(2 * rp + j, RT - 1)) * KT);
                const uint8_t* sf_src = a.wtiles + (size_t)tile * a.rec_bytes + a.codes_bytes;
                for (int kt = 0; kt < KT; ++kt, ++n) {
                    if (n >= S && !dead && !mbar_wait(&empty_bar[s], ph ^ 1, a.status, KID_TCP, 1 + j)) dead = true;
                    uint8_t* st = ring + s * Cfg::STAGE;
                    if (warp_elect()) {
                        // TMA counts the bytes it reads: 8192 for a packed FP4 tile that fills 16384 of shared memory
                        mbar_expect_tx(&full_bar[s], (FMT == FMT_FP4 ? 8192 : 16384) + (WMX ? 512 : 0) + (j == 0 ? NTOK * 128 : 0));
                        tma_3d_nh(st + j * Cfg::A_BYTES, &a.tm_w, 0, 0, tile, &full_bar[s]);
                        if (WMX) bulk_g2s(st + Cfg::SFA_OFF + j * 512, sf_src, 512, &full_bar[s], pol);
                        if (j == 0) tma_2d(st + Cfg::B_OFF, &a.tm_x, kt * 128, xrow0, &full_bar[s], pol);
                    }
                    __syncwarp();
                    if (j == 1) {
#pragma unroll
                        for (int t = lane; t < NTOK; t += 32) {
                            // MX: the token's 4 UE8M0 bytes of this K tile go to its row of the scale atom; DS: its fp32 scale
                            const uint32_t* src = (const uint32_t*)a.xscale + (size_t)min(xrow0 + t, a.x_rows - 1) * KT + kt;
                            if (AMX) cp_async4(st + Cfg::SFB_OFF + (t & 31) * 16 + (t >> 5) * 4, src);
                            else cp_async4(s_xs + (n & (XR - 1)) * NTOK + t, src);
                        }
                        cp_async_arrive_noinc(&full_bar[s]);
                    }
                    ++tile;
                    sf_src += a.rec_bytes;
                    if (++s == S) { s = 0; ph ^= 1; }
                }
            }
        }
    } else if (warp == 1 || warp == 3) {
        // ================= MMA issuers: issuer j multiplies row tile j of every stage into accumulator j =================
        // The whole warp runs the loop and one elected lane issues (tcgen05 operands are uniform-register operands).
        const int j = warp >> 1;
        if (ibeg < iend) {
            const uint32_t tmu = warp_uniform(tm);
            const uint64_t ad0 = warp_uniform(tc_smem_desc(ring + j * Cfg::A_BYTES, 16, 1024, 2)),
                           bd0 = warp_uniform(tc_smem_desc(ring + Cfg::B_OFF, 16, 1024, 2));
            const uint64_t fa0 = warp_uniform(tc_smem_desc(ring + Cfg::SFA_OFF + j * 512, 512, 128, 0)),
                           fb0 = warp_uniform(tc_smem_desc(ring + Cfg::SFB_OFF, 512, 128, 0));
            const uint32_t ones_a = tmu + Cfg::TM_SFA + 4 * (2 * S + j), ones_b = tmu + Cfg::TM_SFB + 4 * (2 * S + j);
            if (!AMX) {
                const uint64_t ones_d = warp_uniform(tc_smem_desc(ring + Cfg::ONES_OFF, 512, 128, 0));  // shuffles: outside the election
                if (warp_elect()) {
                    tc_cp_sf(ones_b, ones_d);
                    if (!WMX) tc_cp_sf(ones_a, ones_d);
                }
                __syncwarp();
            }
            int s = 0;
            uint32_t ph = 0;
            int nit = 0, n = 0;
            int acc_i = j;  // MX: issuer j keeps accumulator j for the whole K
            for (int it = ibeg; it < iend; it += G) {
                // the MMA's N follows the rows the slot really holds (a multiple of 16): the last tile of an expert is
                // rarely full, and a 48-column MMA takes 60 cycles where a 128-column one takes 97
                int slot, rp;
                item_of(it, slot, rp);
                const int cnt = slot_of(slot).z;
                if (cnt <= 0) continue;
                const uint32_t idesc = tc_idesc_mx(cnt > NTOK - 16 ? NTOK : cnt <= 16 ? 16 : (cnt + 15) & ~15, FMT == FMT_FP4);
                if (AMX) {
                    // the accumulator is single-buffered: wait until the epilogue has drained the previous item
                    if (nit > 0 && !dead && !mbar_wait(&tempty_bar[3 * j], (uint32_t)((nit - 1) & 1), a.status, KID_TCP, 3)) dead = true;
                    tc_fence_after();
                }
                for (int kt = 0; kt < KT; ++kt, ++n) {
                    if (!dead && !mbar_wait(&full_bar[s], ph, a.status, KID_TCP, 4)) dead = true;
                    if (AMX) {
                        fence_proxy_async();  // the activation scale atom was written by cp.async (generic proxy)
                    } else {
                        // per-tile promotion: the two issuers rotate over three accumulators (use g = 2n + j takes accumulator
                        // g % 3), so one is being read out while the other two take MMAs; wait for its previous reader
                        // Barriers are per (accumulator, issuer): that pair recurs every 6 uses, always with the same
                        // committing issuer and the same reading epilogue group, so the phases of a barrier are consumed in
                        // order by one party (a parity wait cannot tell phase p from p + 2).  The previous user of the
                        // accumulator, use g - 3, is the other issuer's.
                        const int g = 2 * n + j;
                        acc_i = g % 3;
                        if (g >= 3 && !dead && !mbar_wait(&tempty_bar[acc_i * 2 + (j ^ 1)], (uint32_t)(((g - 3) / 6) & 1), a.status, KID_TCP, 3)) dead = true;
                        tc_fence_after();
                    }
                    const uint64_t so = (uint64_t)((s * Cfg::STAGE) >> 4);
                    const uint32_t d = tmu + acc_i * NTOK;
                    if (warp_elect()) {
                        // each issuer keeps its own copy of the stage's scales in tensor memory
                        uint32_t sfa = ones_a, sfb = ones_b;
                        if (WMX) { sfa = tmu + Cfg::TM_SFA + 4 * (2 * s + j); tc_cp_sf(sfa, fa0 + so); }
                        if (AMX) { sfb = tmu + Cfg::TM_SFB + 4 * (2 * s + j); tc_cp_sf(sfb, fb0 + so); }
#pragma unroll
                        for (int kc = 0; kc < 4; ++kc)
                            tc_mma_mx(d, ad0 + so + (uint64_t)(kc * 2), bd0 + so + (uint64_t)(kc * 2), tc_idesc_sf(idesc, kc), sfa, sfb,
                                      ((!AMX || kt == 0) && kc == 0) ? 0u : 1u);
                        tc_commit(&empty_bar[s]);
                        if (!AMX || kt + 1 == KT) tc_commit(&tfull_bar[acc_i * 2 + j]);
                    }
                    __syncwarp();
                    if (++s == S) { s = 0; ph ^= 1; }
                }
                ++nit;
            }
        }
    } else if (warp >= Cfg::EPI_WARP0) {
        // ================= epilogue warps (thread = weight row of the tile = tensor-memory lane) =================
        const int e = warp - Cfg::EPI_WARP0;
        const int ga = e >> 3;                 // accumulator = row tile of the pair
        const int cb = ((e >> 2) & 1) * CPT;   // first of this thread's CPT token columns
        const int q4 = warp & 3;               // tensor-memory lane quadrant this warp may read
        const int r = 32 * q4 + lane;
        const uint32_t tlane = tm + ((uint32_t)(32 * q4) << 16) + cb;  // + NTOK * accumulator
        float acc[CPT];
        int nit = 0, n = 0;
        for (int it = ibeg; it < iend; it += G) {
            int slot, rp;
            item_of(it, slot, rp);
            const int rt = 2 * rp + ga;
            const int4 sl = slot_of(slot);
            const int xrow0 = sl.y, cnt = sl.z;
            if (cnt <= 0) continue;
            float rw0 = 0.f, rw1 = 0.f;
            if (EPI == EPI_W13 && AMX) {
                // routing weights of this thread's token columns, one per lane, fetched while the item's MMAs run
                rw0 = (cb + lane < cnt) ? __ldg(a.row_w + xrow0 + cb + lane) : 0.f;
                if (CPT > 32) rw1 = (cb + 32 + lane < cnt) ? __ldg(a.row_w + xrow0 + cb + 32 + lane) : 0.f;
            }
            if (AMX) {
                if (!dead && !mbar_wait(&tfull_bar[3 * ga], (uint32_t)(nit & 1), a.status, KID_TCP, 5)) dead = true;
                tc_fence_after();
#pragma unroll
                for (int c0 = 0; c0 < CPT; c0 += 32) tmem_ld<32>(tlane + ga * NTOK + c0, acc + c0);
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(&tempty_bar[3 * ga]);
            } else {
#pragma unroll
                for (int j = 0; j < CPT; ++j) acc[j] = 0.f;
                for (int kt = 0; kt < KT; ++kt, ++n) {
                    // DS weights: the tile's fp32 128x128 block scale, fetched before the wait
                    const float wds = WMX ? 1.0f : __ldg(a.wscale_ds + (size_t)min(rt, RT - 1) * KT + kt);
                    const int g = 2 * n + ga, ai = g % 3;
                    if (!dead && !mbar_wait(&tfull_bar[ai * 2 + ga], (uint32_t)((g / 6) & 1), a.status, KID_TCP, 5)) dead = true;
                    tc_fence_after();
                    const float* xs = s_xs + (n & (XR - 1)) * NTOK + cb;
                    constexpr int CH = CPT == 32 ? 32 : 16;  // columns in flight per load: what the registers allow
                    // (every chunk is read back even where a ragged last tile leaves columns empty: bounding the loop by
                    // the slot's row count made the grouped DS GEMMs 25 % slower, 11.5 -> 14.4 ms)
#pragma unroll
                    for (int c0 = 0; c0 < CPT; c0 += CH) {
                        float v[CH];
                        tmem_ld<CH>(tlane + ai * NTOK + c0, v);
                        if (c0 == CPT - CH) {
                            // everything is in registers: hand the accumulator back before the arithmetic
                            tc_fence_before();
                            __syncwarp();
                            if (lane == 0) mbar_arrive(&tempty_bar[ai * 2 + ga]);
                        }
#pragma unroll
                        for (int j = 0; j < CH; j += 4) {
                            // two columns per instruction (packed fp32: same roundings as the scalar mul / fma)
                            float4 t4 = *(const float4*)(xs + c0 + j);
                            if (!WMX) {
                                mul_f32x2(t4.x, t4.y, wds, wds);
                                mul_f32x2(t4.z, t4.w, wds, wds);
                            }
                            fma_f32x2(acc[c0 + j], acc[c0 + j + 1], v[j], v[j + 1], t4.x, t4.y);
                            fma_f32x2(acc[c0 + j + 2], acc[c0 + j + 3], v[j + 2], v[j + 3], t4.z, t4.w);
                        }
                    }
                }
            }
            if (EPI == EPI_W13 && !AMX) {
                // (per-tile promotion keeps 64 accumulators and 16 loaded columns live: no registers to spare in the K loop)
                rw0 = (cb + lane < cnt) ? __ldg(a.row_w + xrow0 + cb + lane) : 0.f;
                if (CPT > 32) rw1 = (cb + 32 + lane < cnt) ? __ldg(a.row_w + xrow0 + cb + 32 + lane) : 0.f;
            }
            if (EPI == EPI_W13 || (EPI == EPI_DENSE && a.swiglu)) {
                // (EPI_DENSE with the SwiGLU option: the FP8 shared expert's gate/up weight, no routing weight)
                // lanes l and l^8 hold a gate row and its up row (rows 0..7 / 8..15 of every 16-row group); after the
                // exchange the gate lane finishes column j, the up lane column j + 1.
                // SwiGLU as crates/kernels/cu/gemv.cu:470-483: bf16 rounds, optional clamp, routing weight folded in
                bf16* ocol = (bf16*)a.out + rt * 64 + (r >> 4) * 8 + (r & 7);
                const float L = a.swiglu_limit;
                const bool is_gate = (r & 8) == 0;
#pragma unroll
                for (int j = 0; j < CPT; j += 2) {
                    const float o0 = __shfl_xor_sync(0xffffffffu, acc[j], 8);
                    const float o1 = __shfl_xor_sync(0xffffffffu, acc[j + 1], 8);
                    const int col = is_gate ? j : j + 1;
                    const float rw = EPI == EPI_W13 ? __shfl_sync(0xffffffffu, j < 32 ? rw0 : rw1, col & 31) : 1.0f;
                    if (cb + col < cnt && rt < RT) {   // (rt == RT: the repeated tile of an odd row-tile count)
                        const int row = xrow0 + cb + col;
                        float gt = bf16_round(is_gate ? acc[j] : o1), up = bf16_round(is_gate ? o0 : acc[j + 1]);
                        if (L > 0.f) { up = fminf(fmaxf(up, -L), L); gt = fminf(gt, L); }
                        const float val = gt / (1.0f + expf(-gt)) * up * rw;
                        ocol[(size_t)row * a.ldo] = __float2bfloat16(val);
                    }
                }
            } else if (EPI == EPI_DENSE) {
                const int col = rt * 128 + r;
#pragma unroll
                for (int j = 0; j < CPT; ++j)
                {
                    const float v = acc[j] * a.alpha;
                    const bool mine = cb + j < cnt && col < a.n_rows;
                    if (a.rope_cos) {
                        const float pv = __shfl_xor_sync(0xffffffffu, v, 1);   // row ^ 1 is the neighbouring lane
                        if (mine) dense_store_rope(a, xrow0 + cb + j, col, v, pv);
                    } else if (mine) {
                        dense_store(a, xrow0 + cb + j, col, v);
                    }
                }
            } else {
                float* o = (float*)a.out;
                const int col = rt * 128 + r;
#pragma unroll
                for (int j = 0; j < CPT; ++j)
                    if (cb + j < cnt && col < a.n_rows) o[(size_t)(xrow0 + cb + j) * a.ldo + col] = acc[j];
            }
            ++nit;
        }
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    if (warp == 1) tmem_dealloc(tm, Cfg::TM_COLS);
}

}  // namespace dsuf
