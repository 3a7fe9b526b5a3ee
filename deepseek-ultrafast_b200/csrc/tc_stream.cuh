// tcgen05 weight-streaming kernel for decode shapes ("swap-AB": the 128 weight rows of a tile are the MMA's M, the
// few token rows its N), same work decomposition as stream_gemv.cuh but with ZERO per-weight-element instructions:
//   * TMA lands the weight tile in shared memory in the tensor core's operand layout (FP4 tiles are widened to
//     8-bit containers by the TMA unit itself, CU_TENSOR_MAP_DATA_TYPE_16U4_ALIGN16B);
//   * tcgen05.mma kind::mxf8f6f4.block_scale, 4 x K=32 per 128-K tile; UE8M0 weight scales are applied by the tensor
//     core from tensor memory (tcgen05.cp of the tile record's 512-byte scale atom);
//   * accumulators live in tensor memory; four epilogue warps read them back.  With MX (power-of-two) activation
//     scales the whole K accumulates in tensor memory; with DS (fp32 per 128-K) activation / weight scales each
//     128-K tile is promoted into fp32 registers with its scale pair, on a 4-deep ring of accumulators.
//   * Measured on B200: the thread that issues the tcgen05 instructions is the serial resource of this kernel
//     (~75 cycles per MMA of issue back-pressure plus the scale copy and the commit).  In the per-tile (DS) mode
//     two warps therefore issue alternate tiles, each into its own accumulator-ring entries.
// Replaces tc_gemv_fp8 (crates/kernels/cu/tcgemv.cu:33-241) and the mma.sync decode MoE
// (cu/gemv.cu:1016-1692).  The reference's tcgen05 decode kernels load a CTA's whole K slice up front and then
// drain it; here the ring is refilled continuously across row tiles and experts.
#pragma once
#include <cuda.h>
#include "stream_gemv.cuh"

namespace dsuf {

constexpr int KID_TC = 3;
// warp 0: weight producer, 1: MMA issuer A, 2-5: epilogue, 6: activation producer, 7: MMA issuer B,
// 8 / 9: second weight / activation producer, 10-13: second epilogue group, 14 / 15: MMA issuers C / D
// (token tiles up to 16 columns)
constexpr int TC_EPI_THREADS = 128;

// PAIR: tile records (128-K tiles) per ring stage.  With two, every hand-off of the pipeline (stage full / stage free /
// accumulator full / accumulator free) moves 256 K of a weight row tile instead of 128: half the barrier round trips
// per byte, which is what bounds the 8.7 KB FP4 tiles (the tensor pipe and TMA are far from busy).
template <int N, int PAIR = 1>
struct TcCfg {
    static constexpr int A1 = 16384;                                 // one weight tile in 8-bit containers
    static constexpr int B1 = N * 128 < 1024 ? 1024 : N * 128;       // N token rows of 128 bytes of one K tile
    static constexpr int A_BYTES = A1 * PAIR;
    static constexpr int B_BYTES = B1 * PAIR;
    static constexpr int B_OFF = A_BYTES;
    static constexpr int SFA_OFF = B_OFF + B_BYTES;          // weight scale atoms (512 each)
    static constexpr int SFB_OFF = SFA_OFF + 512 * PAIR;     // MX activations: activation scale atoms (512 each)
    static constexpr int STAGE = A_BYTES + B_BYTES + 1024 * PAIR;
    static constexpr int NE = N <= 16 ? 2 : 1;        // epilogue warp groups (per-tile mode: alternate tiles)
    static constexpr int RED_BYTES = NE == 2 ? 2 * N * 128 * 4 : 0;  // static shared memory of the group combine
    static constexpr int S_FIT = (226 * 1024 - 2048 - RED_BYTES) / STAGE;
    // A multiple of the number of issuers (4 for N <= 16, else 2), so that every stage is always handled by the
    // same issuer: a parity wait cannot tell phase p from phase p + 2, and only the issuer that consumed phase p - 1
    // of a stage is certain not to reach the wait before phase p has begun.
    static constexpr int NISSUE = (N <= 16 && PAIR == 1) ? 4 : 2;   // issuer warps dealing stages round-robin
    static constexpr int STAGES = (S_FIT > 12 ? 12 : S_FIT) & ~(NISSUE - 1);
    static constexpr int ONES_OFF = STAGE * STAGES;  // 512-byte atom of UE8M0 1.0
    static constexpr int SMEM = STAGE * STAGES + 512 + 1024;
    static constexpr int ACC_COLS = N * PAIR;        // tensor-memory columns of one accumulator-ring entry (per-tile mode)
    // accumulator ring (a power of two); with two tiles per entry eight entries are as deep as sixteen single ones, and the
    // shorter scale ring that goes with them keeps the static shared memory inside the budget
    static constexpr int NB = PAIR == 2 ? (ACC_COLS <= 32 ? 8 : ACC_COLS <= 64 ? 4 : 2) : ACC_COLS <= 16 ? 16 : ACC_COLS <= 32 ? 8 : ACC_COLS <= 64 ? 4 : 2;
    // producer warps per kind (weights / activations), tiles dealt round-robin: a producer spends ~1100 cycles per tile
    // of its own (two barrier waits, the copies, the scale gathers); four of each kind measured no faster than two
    static constexpr int NP = 2;
    static constexpr int THREADS = 512;  // 16 warps
    static constexpr int TM_SFA = 256, TM_SFB = 384, TM_COLS = 512;
    static_assert(NB * ACC_COLS <= 256 && STAGES >= 4 && N <= 128, "tensor-memory / shared-memory budget");
};


template <int FMT, int WMX, int AMX, int N, int EPI, int PAIR = 1>
__global__ void __launch_bounds__(TcCfg<N, PAIR>::THREADS, 1) tc_stream_kernel(const __grid_constant__ StreamArgs a) {
    using Cfg = TcCfg<N, PAIR>;
    constexpr bool PER_TILE = (AMX == 0);   // promote every 128-K tile with fp32 scales
    constexpr int S = Cfg::STAGES, ACC_COLS = PER_TILE ? Cfg::ACC_COLS : N;
    constexpr int A1 = Cfg::A1, B1 = Cfg::B1;
    // MMA-issuing warps of the per-tile mode: an issuer spends ~600 cycles per tile of its own (waits, fences, scale
    // copies, commits around 4 MMAs), so narrow token tiles (180 cycles of MMA per tile) take four to keep up with HBM
    constexpr int NI = PER_TILE ? Cfg::NISSUE : 1;
    // whole-K mode with token tiles up to 64 columns: several issuers as well (four up to 16 columns, else two), tiles
    // dealt round-robin, each accumulating into its own part of the ring entry; the epilogue adds the parts
    constexpr bool DUAL_WHOLE = !PER_TILE && N <= 64;
    constexpr int NIW = !DUAL_WHOLE ? 1 : Cfg::NISSUE;
    constexpr int ACCW = NIW * ACC_COLS;  // tensor-memory columns of one ring entry
    static_assert(S % NI == 0 && S % NIW == 0 && S % Cfg::NP == 0, "stage ownership must not rotate among issuers or producers (parity waits alias)");
    constexpr int NB = Cfg::NB * ACCW > 256 ? 256 / ACCW : Cfg::NB;  // ring entries in use (a power of two)
    static_assert(NB * ACCW <= 256, "accumulator ring overlaps the scale columns");
    constexpr int NP = Cfg::NP;
    // epilogue groups actually working: the second group pays off where tiles are 8.7 KB (FP4 experts), not for dense FP8
    constexpr int NE = (PER_TILE && Cfg::NE == 2 && EPI != EPI_DENSE) ? 2 : 1;
    // wide token tiles: the two epilogue groups split the token COLUMNS of every accumulator instead
    constexpr bool CSPLIT = N >= 32;
    constexpr int NC = CSPLIT ? N / 2 : N;            // columns per epilogue thread
    constexpr int EG1 = 10;                           // first warp of the second epilogue group
    constexpr int EPI_BAR = CSPLIT ? 256 : 128;       // threads meeting at the dense stream-K fix-up
    extern __shared__ uint8_t smem_raw[];
    uint8_t* ring = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    __shared__ __align__(8) uint64_t full_bar[S], empty_bar[S], tfull_bar[NB], tempty_bar[NB];
    static_assert((NB & (NB - 1)) == 0, "accumulator ring size must be a power of two");
    __shared__ uint32_t s_tmem;
    __shared__ int s_flag;
    // DS scales outlive the stage (the epilogue reads them after the MMAs completed).  A ring of XR >= S + NB entries
    // indexed by tile number needs no barrier of its own: a producer writing tile n has seen the MMAs of tile n - S
    // complete, which were issued only after the epilogue had released the accumulator of tile n - S - NB, and the
    // epilogue reads a tile's scales before it releases its accumulator.
    constexpr int XSE = 4 * N * PAIR + (WMX ? 0 : 16);  // entry: N activation scales per K tile (+ the tiles' weight scales, DS weights)
    constexpr int XR = S + NB <= 16 ? 16 : 32;
    static_assert(S + NB <= XR, "scale ring shorter than stages + accumulators");
    __shared__ __align__(16) uint8_t s_xs[XR * XSE];
    __shared__ float s_red[Cfg::NE == 2 ? 2 * N * 128 : 1];  // second epilogue group -> first, double buffered by item

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int G = gridDim.x, c = blockIdx.x;
    const int RT = a.RT;
    const int KT = a.KT / PAIR;   // ring steps per item: PAIR K tiles each (the launcher checks that the K tile count divides)
    const int KTT = a.KT;         // K tiles per item (row stride of the scale arrays and of the tile sequence)
    bool dead = false;  // set by the first expired wait: nothing is waited for again, the loops stay finite

    if (warp == 1) {
        tmem_alloc(&s_tmem, Cfg::TM_COLS);
        tmem_relinquish();
    }
    if (tid == 0) {
        for (int s = 0; s < S; ++s) {
            mbar_init(&full_bar[s], 2 + 32);  // weight expect_tx + activation expect_tx + 32 cp.async lanes
            mbar_init(&empty_bar[s], 1);  // tcgen05.commit: the tensor core has finished reading the stage
        }
        for (int b = 0; b < NB; ++b) {
            mbar_init(&tfull_bar[b], NIW);
            mbar_init(&tempty_bar[b], CSPLIT ? 8 : 4);
        }
        mbar_fence_init();
    }
    if (tid >= 64 && tid < 192) ((uint32_t*)(ring + Cfg::ONES_OFF))[tid - 64] = 0x7f7f7f7fu;  // one atom of UE8M0 1.0
    fence_proxy_async();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tm = s_tmem;
    pdl_wait();
    pdl_launch_dependents();  // dependents still wait for this grid to finish; only their prologues overlap

    // ---- this CTA's span of the global tile sequence (see stream_gemv.cuh) ----
    long long beg, end;
    // cluster K-split (dense weights with few row tiles): cluster r owns row tile r, its CTA j the K tiles
    // [j KT / cs, (j + 1) KT / cs); the partial sums meet through distributed shared memory, every CTA of the cluster
    // summing and storing its share of the token columns
    const int ksl = EPI == EPI_DENSE ? a.kslices : 0;
    const int krank = ksl > 1 ? (int)cluster_cta_rank() : 0;
    bool cluster_done = false;  // this warp has been through the two cluster barriers of the reduce
    if (EPI == EPI_DENSE && ksl > 0) {
        const int rt_c = c / ksl;
        beg = (long long)rt_c * KT + (long long)krank * KT / ksl;
        end = (long long)rt_c * KT + (long long)(krank + 1) * KT / ksl;
    } else if (EPI == EPI_DENSE && a.whole_items) {
        beg = ((long long)c * RT / G) * KT;
        end = ((long long)(c + 1) * RT / G) * KT;
    } else if (EPI == EPI_DENSE) {
        const long long tot = (long long)RT * KT;
        beg = (long long)c * tot / G;
        end = (long long)(c + 1) * tot / G;
    } else {
        const long long q = (long long)(*a.nslots) * RT;
        beg = ((long long)c * q / G) * KT;
        end = ((long long)(c + 1) * q / G) * KT;
    }

    if (warp == 0 || warp == 8) {
        // ================= weight producers (tiles dealt round-robin): tile codes + scale atom =================
        const int pj = warp == 0 ? 0 : 1;
        // The whole warp runs the loop (so every value stays warp-uniform and the TMA descriptors live in uniform
        // registers); one elected lane issues.
        if (pj < NP && beg + pj < end) {
            if (lane == 0) prefetch_tmap(&a.tm_w);
            const uint64_t pol_w = policy_evict_first();
            long long q = (beg + pj) / KT;
            int kt = (int)(beg + pj - q * KT);
            int tile = 0;
            const uint8_t* sf_src = nullptr;
            bool fresh = true;
            int s = pj;
            uint32_t ph = 0;
            uint8_t* st = ring + pj * Cfg::STAGE;
            // TMA counts the bytes it READS: a packed FP4 tile is 8192 bytes although it fills 16384 of shared memory
            constexpr uint32_t W_TX = PAIR * ((FMT == FMT_FP4 ? 8192 : 16384) + (WMX ? 512 : 0));
            for (long long i = beg + pj; i < end; i += NP) {
                if (fresh) {
                    long long wbase;
                    if (EPI == EPI_DENSE) {
                        wbase = q * KTT;
                    } else {
                        const int slot = (int)(q / RT);
                        const int rt = (int)(q - (long long)slot * RT);
                        wbase = ((long long)a.slots[slot].x * RT + rt) * KTT;
                    }
                    tile = (int)(wbase + kt * PAIR);
                    sf_src = a.wtiles + (size_t)tile * a.rec_bytes + a.codes_bytes;
                    fresh = false;
                }
                if (i - beg >= S && !dead && !mbar_wait(&empty_bar[s], ph ^ 1, a.status, KID_TC, 1)) dead = true;
                if (warp_elect()) {
                    mbar_expect_tx(&full_bar[s], W_TX);
#pragma unroll
                    for (int pp = 0; pp < PAIR; ++pp) {
                        tma_3d(st + pp * A1, &a.tm_w, 0, 0, tile + pp, &full_bar[s], pol_w);
                        if (WMX) bulk_g2s(st + Cfg::SFA_OFF + pp * 512, sf_src + (size_t)pp * a.rec_bytes, 512, &full_bar[s], pol_w);
                    }
                }
                __syncwarp();
                tile += NP * PAIR;
                sf_src += (size_t)(NP * PAIR) * a.rec_bytes;
                s += NP;
                st += NP * Cfg::STAGE;
                if (s >= S) { s -= S; st -= S * Cfg::STAGE; ph ^= 1; }
                kt += NP;
                while (kt >= KT) { kt -= KT; ++q; fresh = true; }
            }
        }
    } else if (warp == 6 || warp == 9) {
        // ================= activation producers: token rows by TMA, their block scales by 4-byte async copies =================
        const int pj = warp == 6 ? 0 : 1;
        if (pj < NP && beg + pj < end) {
            if (lane == 0) prefetch_tmap(&a.tm_x);
            const uint64_t pol_x = policy_evict_last();
            long long q = (beg + pj) / KT;
            int kt = (int)(beg + pj - q * KT);
            int xrow0 = 0;
            const float* ws_src = nullptr;
            bool fresh = true;
            int s = pj;
            uint32_t ph = 0;
            uint8_t* st = ring + pj * Cfg::STAGE;
            for (long long i = beg + pj; i < end; i += NP) {
                if (fresh) {
                    int rt;
                    if (EPI == EPI_DENSE) {
                        rt = (int)q;
                        xrow0 = 0;
                    } else {
                        const int slot = (int)(q / RT);
                        rt = (int)(q - (long long)slot * RT);
                        xrow0 = a.slots[slot].y;
                    }
                    ws_src = (!WMX && lane == 31) ? a.wscale_ds + (size_t)rt * KTT : nullptr;
                    fresh = false;
                }
                if (i - beg >= S && !dead && !mbar_wait(&empty_bar[s], ph ^ 1, a.status, KID_TC, 5)) dead = true;
                if (warp_elect()) {
                    mbar_expect_tx(&full_bar[s], PAIR * N * 128);
#pragma unroll
                    for (int pp = 0; pp < PAIR; ++pp)
                        tma_2d(st + Cfg::B_OFF + pp * B1, &a.tm_x, (kt * PAIR + pp) * 128, xrow0, &full_bar[s], pol_x);
                }
                __syncwarp();
                uint8_t* xe = nullptr;
                if (PER_TILE) {
                    // fp32 scales go to the tile's entry of the scale ring (free by construction, see s_xs)
                    xe = s_xs + ((int)(i - beg) & (XR - 1)) * XSE;
                }
#pragma unroll
                for (int n = lane; n < N; n += 32) {
                    // MX: the token's 4 UE8M0 bytes go to its row of the scale atom; DS: its fp32 scale
                    const uint32_t* src = (const uint32_t*)a.xscale + (size_t)min(xrow0 + n, a.x_rows - 1) * KTT + kt * PAIR;
#pragma unroll
                    for (int pp = 0; pp < PAIR; ++pp)
                        cp_async4(AMX ? st + Cfg::SFB_OFF + pp * 512 + (n & 31) * 16 + (n >> 5) * 4 : xe + 4 * (pp * N + n), src + pp);
                }
                if (!WMX && lane == 31) {
#pragma unroll
                    for (int pp = 0; pp < PAIR; ++pp) cp_async4(xe + 4 * N * PAIR + 4 * pp, ws_src + kt * PAIR + pp);
                }
                cp_async_arrive_noinc(&full_bar[s]);
                s += NP;
                st += NP * Cfg::STAGE;
                if (s >= S) { s -= S; st -= S * Cfg::STAGE; ph ^= 1; }
                kt += NP;
                while (kt >= KT) { kt -= KT; ++q; fresh = true; }
            }
        }
    } else if (warp == 1 || warp == 7 || ((NI == 4 || NIW == 4) && (warp == 14 || warp == 15))) {
        // ================= MMA issuers (one thread each; issuer B only in the per-tile mode) =================
        const int j = warp == 1 ? 0 : warp == 7 ? 1 : warp - 12;
        // The whole warp runs the loop and one elected lane issues: tcgen05 operands are uniform-register operands,
        // and a loop run by a single lane of a diverged warp pays a register-file round trip for each of them.
        if (DUAL_WHOLE) {
            if (beg < end) {
                // Every issuer walks every tile of the span (so all know the group boundaries); issuer j issues the tiles
                // j, j + NIW, ... into columns [j*N, (j+1)*N) of the ring entry.  tfull needs all of them: a commit from
                // an issuer that contributed MMAs, a plain arrival from one that did not.
                const uint32_t tmu = warp_uniform(tm);
                const uint32_t idesc = tc_idesc_mx(N, FMT == FMT_FP4);
                const uint32_t ones_a = tmu + Cfg::TM_SFA + 4 * (S * PAIR + j), ones_b = tmu + Cfg::TM_SFB + 4 * (S * PAIR + j);
                const uint64_t ones_d = warp_uniform(tc_smem_desc(ring + Cfg::ONES_OFF, 512, 128, 0));
                if (warp_elect()) {
                    if (!WMX) tc_cp_sf(ones_a, ones_d);
                    if (!AMX) tc_cp_sf(ones_b, ones_d);
                }
                __syncwarp();
                const uint64_t ad0 = warp_uniform(tc_smem_desc(ring, 16, 1024, 2)), bd0 = warp_uniform(tc_smem_desc(ring + Cfg::B_OFF, 16, 1024, 2));
                const uint64_t fa0 = warp_uniform(tc_smem_desc(ring + Cfg::SFA_OFF, 512, 128, 0)),
                               fb0 = warp_uniform(tc_smem_desc(ring + Cfg::SFB_OFF, 512, 128, 0));
                int kt = (int)(beg % KT);
                int s = 0, gidx = 0;
                uint32_t ph = 0;
                bool issued = false, entry_free = false;
                for (long long i = beg; i < end; ++i) {
                    const bool mine = ((int)(i - beg) & (NIW - 1)) == j;
                    const bool group_end = kt + 1 == KT || i + 1 == end;
                    const int b = gidx & (NB - 1);
                    if ((mine || group_end) && !entry_free) {
                        // also before a bare arrival: the entry's previous phase must be complete before this one is fed
                        if (gidx >= NB && !dead && !mbar_wait(&tempty_bar[b], ((gidx / NB) - 1) & 1, a.status, KID_TC, 3)) dead = true;
                        entry_free = true;
                    }
                    if (mine) {
                        if (!dead && !mbar_wait(&full_bar[s], ph, a.status, KID_TC, 2)) dead = true;
                        tc_fence_after();
                        if (AMX) fence_proxy_async();  // the activation scale atom was written by cp.async (generic proxy)
                        const uint64_t so = (uint64_t)((s * Cfg::STAGE) >> 4);
                        if (warp_elect()) {
                            const uint32_t d = tmu + b * ACCW + j * N;
#pragma unroll
                            for (int pp = 0; pp < PAIR; ++pp) {
                                uint32_t sfa = ones_a, sfb = ones_b;
                                if (WMX) { sfa = tmu + Cfg::TM_SFA + 4 * (s * PAIR + pp); tc_cp_sf(sfa, fa0 + so + (uint64_t)(pp * 32)); }
                                if (AMX) { sfb = tmu + Cfg::TM_SFB + 4 * (s * PAIR + pp); tc_cp_sf(sfb, fb0 + so + (uint64_t)(pp * 32)); }
#pragma unroll
                                for (int kc = 0; kc < 4; ++kc)
                                    tc_mma_mx(d, ad0 + so + (uint64_t)(pp * (A1 >> 4) + kc * 2), bd0 + so + (uint64_t)(pp * (B1 >> 4) + kc * 2),
                                              tc_idesc_sf(idesc, kc), sfa, sfb, (!issued && pp == 0 && kc == 0) ? 0u : 1u);
                            }
                            tc_commit(&empty_bar[s]);
                            if (group_end) tc_commit(&tfull_bar[b]);
                        }
                        issued = true;
                    } else if (group_end) {
                        if (warp_elect()) {
                            if (issued) tc_commit(&tfull_bar[b]);
                            else mbar_arrive(&tfull_bar[b]);
                        }
                    }
                    __syncwarp();
                    if (group_end) { ++gidx; issued = false; entry_free = false; }
                    if (++kt == KT) kt = 0;
                    if (++s == S) { s = 0; ph ^= 1; }
                }
            }
        } else if (j < NI && beg + j < end) {
            const uint32_t tmu = warp_uniform(tm);
            const uint32_t idesc = tc_idesc_mx(N, FMT == FMT_FP4);
            const uint32_t ones_a = tmu + Cfg::TM_SFA + 4 * (S * PAIR + j), ones_b = tmu + Cfg::TM_SFB + 4 * (S * PAIR + j);
            const uint64_t ones_d = warp_uniform(tc_smem_desc(ring + Cfg::ONES_OFF, 512, 128, 0));
            if (warp_elect()) {
                if (!WMX) tc_cp_sf(ones_a, ones_d);
                if (!AMX) tc_cp_sf(ones_b, ones_d);
            }
            __syncwarp();
            // descriptors of stage 0; a stage is selected by adding its byte offset / 16 to the address field
            const uint64_t ad0 = warp_uniform(tc_smem_desc(ring, 16, 1024, 2)), bd0 = warp_uniform(tc_smem_desc(ring + Cfg::B_OFF, 16, 1024, 2));
            const uint64_t fa0 = warp_uniform(tc_smem_desc(ring + Cfg::SFA_OFF, 512, 128, 0)),
                           fb0 = warp_uniform(tc_smem_desc(ring + Cfg::SFB_OFF, 512, 128, 0));
            long long q = beg / KT;
            int kt = (int)(beg - q * KT);
            int s = j, gidx = 0;
            uint32_t ph = 0;
            bool group_open = false;
            for (long long i = beg + j; i < end; i += NI) {
                if (!dead && !mbar_wait(&full_bar[s], ph, a.status, KID_TC, 2)) dead = true;
                tc_fence_after();
                if (AMX) fence_proxy_async();  // the activation scale atom was written by cp.async (generic proxy)
                int b;
                bool first_of_group;
                if (PER_TILE) {
                    const int n = (int)(i - beg);
                    b = n & (NB - 1);
                    first_of_group = true;
                    if (n >= NB && !dead && !mbar_wait(&tempty_bar[b], ((n / NB) - 1) & 1, a.status, KID_TC, 3)) dead = true;
                    tc_fence_after();
                } else {
                    b = gidx % NB;
                    first_of_group = !group_open;
                    if (!group_open) {
                        if (gidx >= NB && !dead && !mbar_wait(&tempty_bar[b], ((gidx / NB) - 1) & 1, a.status, KID_TC, 3)) dead = true;
                        tc_fence_after();
                        group_open = true;
                    }
                }
                const uint64_t so = (uint64_t)((s * Cfg::STAGE) >> 4);
                const bool group_end = PER_TILE || kt + 1 == KT || i + 1 == end;
                if (warp_elect()) {
#pragma unroll
                    for (int pp = 0; pp < PAIR; ++pp) {
                        uint32_t sfa = ones_a, sfb = ones_b;
                        if (WMX) { sfa = tmu + Cfg::TM_SFA + 4 * (s * PAIR + pp); tc_cp_sf(sfa, fa0 + so + (uint64_t)(pp * 32)); }
                        if (AMX) { sfb = tmu + Cfg::TM_SFB + 4 * (s * PAIR + pp); tc_cp_sf(sfb, fb0 + so + (uint64_t)(pp * 32)); }
                        // per-tile mode: every K tile of the stage has its own accumulator columns (promoted with its own scales)
                        const uint32_t d = tmu + b * ACC_COLS + (PER_TILE ? pp * N : 0);
#pragma unroll
                        for (int kc = 0; kc < 4; ++kc)
                            tc_mma_mx(d, ad0 + so + (uint64_t)(pp * (A1 >> 4) + kc * 2), bd0 + so + (uint64_t)(pp * (B1 >> 4) + kc * 2),
                                      tc_idesc_sf(idesc, kc), sfa, sfb, (first_of_group && (PER_TILE || pp == 0) && kc == 0) ? 0u : 1u);
                    }
                    tc_commit(&empty_bar[s]);
                    if (group_end) tc_commit(&tfull_bar[b]);
                }
                __syncwarp();
                if (!PER_TILE) {
                    if (group_end) { ++gidx; group_open = false; }
                    if (++kt == KT) { kt = 0; ++q; }
                }
                s += NI;
                if (s >= S) { s -= S; ph ^= 1; }
            }
        }
    } else if ((warp >= 2 && warp <= 5) || ((NE == 2 || CSPLIT) && warp >= EG1 && warp < EG1 + 4)) {
        // ================= epilogue warps (thread = weight row of the tile = tensor-memory lane) =================
        // per-tile mode with narrow token tiles: two groups of four warps take alternate tiles and add up at item end
        const int eg = warp >= EG1 ? 1 : 0;
        const int cb = CSPLIT ? eg * NC : 0;              // first token column this thread owns
        const int q4 = warp & 3;
        const int r = 32 * q4 + lane;
        const int etid = (warp >= EG1 ? warp - EG1 : warp - 2) * 32 + lane;
        const uint32_t lane_base = (uint32_t)(32 * q4) << 16;
        float acc[NC];
#pragma unroll
        for (int j = 0; j < NC; ++j) acc[j] = 0.f;
        long long q = beg / KT;
        int kt = (int)(beg - q * KT);
        int rt = 0, xrow0 = 0, cnt = 0;
        bool fresh = true;
        int gidx = 0, es = 0, items_done = 0;
        const uint8_t* est = ring;
        long long g0 = beg;  // first tile of the current accumulation group
        float rwreg[(NC + 31) / 32] = {};
        for (long long i = beg; i < end; ++i) {
            if (fresh) {
                if (EPI == EPI_DENSE) {
                    rt = (int)q;
                    xrow0 = 0;
                    cnt = a.m;
                } else {
                    const int slot = (int)(q / RT);
                    rt = (int)(q - (long long)slot * RT);
                    const int4 sl = a.slots[slot];
                    xrow0 = sl.y;
                    cnt = sl.z;
                    if (EPI == EPI_W13) {
                        // routing weights of this thread's token columns, one per lane, fetched while the item's MMAs run
#pragma unroll
                        for (int k = 0; k < (NC + 31) / 32; ++k)
                            rwreg[k] = (cb + 32 * k + lane < cnt) ? __ldg(a.row_w + xrow0 + cb + 32 * k + lane) : 0.f;
                    }
                }
                fresh = false;
            }
            const bool item_end = (kt + 1 == KT) || (i + 1 == end);
            const bool mine = NE == 1 || ((int)(i - beg) & 1) == eg;
            if (!mine) ++gidx;
            if ((PER_TILE || item_end) && mine) {
                const int b = gidx % NB;
                if (!dead && !mbar_wait(&tfull_bar[b], (gidx / NB) & 1, a.status, KID_TC, 4)) dead = true;
                tc_fence_after();
                {
                    float wdsp[PAIR];
#pragma unroll
                    for (int pp = 0; pp < PAIR; ++pp)
                        wdsp[pp] = (PER_TILE && !WMX) ? *(const float*)(s_xs + (gidx & (XR - 1)) * XSE + 4 * N * PAIR + 4 * pp) : 1.0f;
                    constexpr int CH = NC < 32 ? NC : 32;
                    // several issuers in the whole-K mode: part p of the entry holds a sum iff the group, which started at
                    // tile g0 and has gcnt tiles, contains a tile dealt to issuer p; the parts are added in a fixed order
                    const int gcnt = (int)(i - g0) + 1, gph = (int)(g0 - beg) & (NIW - 1);
#pragma unroll
                    for (int c0 = 0; c0 < NC; c0 += CH) {
                        float v[CH];
                        if (DUAL_WHOLE) {
#pragma unroll
                            for (int j = 0; j < CH; ++j) v[j] = 0.f;
#pragma unroll
                            for (int p = 0; p < NIW; ++p) {
                                if (gcnt >= NIW || ((p - gph) & (NIW - 1)) < gcnt) {
                                    float v2[CH];
                                    tmem_ld<CH>(tm + lane_base + b * ACCW + p * N + cb + c0, v2);
#pragma unroll
                                    for (int j = 0; j < CH; ++j) v[j] += v2[j];
                                }
                            }
                        } else if (PAIR == 1) {
                            tmem_ld<CH>(tm + lane_base + b * ACCW + cb + c0, v);
                        }
                        if (PER_TILE) {
                            // the stage's K tiles, each with its own accumulator columns and its own activation scales;
                            // both loads are in flight before the first is waited for
                            float v1[PAIR == 2 ? CH : 1];
                            if (PAIR == 2) {
                                tmem_ld_issue<CH>(tm + lane_base + b * ACCW + cb + c0, v);
                                tmem_ld_issue<CH>(tm + lane_base + b * ACCW + N + cb + c0, v1);
                                tmem_wait_ld();
                            }
#pragma unroll
                            for (int pp = 0; pp < PAIR; ++pp) {
#pragma unroll
                                for (int j = 0; j < CH; j += 4) {
                                    float4 t4 = *(const float4*)(s_xs + (gidx & (XR - 1)) * XSE + 4 * (pp * N + cb + c0 + j));
                                    const float* vv = (PAIR == 2 && pp == 1) ? v1 : v;
                                    const float wds = wdsp[pp];
                                    if constexpr (N >= 32) {
                                        // wide token tiles: two columns per instruction (packed fp32, same roundings)
                                        mul_f32x2(t4.x, t4.y, wds, wds);
                                        mul_f32x2(t4.z, t4.w, wds, wds);
                                        fma_f32x2(acc[c0 + j], acc[c0 + j + 1], vv[j], vv[j + 1], t4.x, t4.y);
                                        fma_f32x2(acc[c0 + j + 2], acc[c0 + j + 3], vv[j + 2], vv[j + 3], t4.z, t4.w);
                                    } else {
                                        acc[c0 + j] = fmaf(vv[j], wds * t4.x, acc[c0 + j]);
                                        acc[c0 + j + 1] = fmaf(vv[j + 1], wds * t4.y, acc[c0 + j + 1]);
                                        acc[c0 + j + 2] = fmaf(vv[j + 2], wds * t4.z, acc[c0 + j + 2]);
                                        acc[c0 + j + 3] = fmaf(vv[j + 3], wds * t4.w, acc[c0 + j + 3]);
                                    }
                                }
                            }
                        } else {
#pragma unroll
                            for (int j = 0; j < CH; ++j) acc[c0 + j] = v[j];
                        }
                    }
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) {
                    mbar_arrive(&tempty_bar[b]);
                }
                ++gidx;
            }
            if (item_end && NE == 2) {
                float* red = s_red + (items_done & 1) * (N * 128);
                if (eg == 1) {
#pragma unroll
                    for (int j = 0; j < N; ++j) red[j * 128 + r] = acc[j];
                }
                named_bar_sync(2, 256);
                if (eg == 0) {
#pragma unroll
                    for (int j = 0; j < N; ++j) acc[j] += red[j * 128 + r];
                }
                ++items_done;
            }
            if (item_end && (eg == 0 || CSPLIT)) {
                // ---------------- flush the item (column-split groups each flush their own token columns) ----------------
                if (EPI == EPI_DENSE) {
                    const long long it0 = q * KT;
                    const bool whole = beg <= it0 && end >= it0 + KT;
                    bool do_store = whole;
                    if (ksl > 1) {
                        // This CTA's only item.  Every CTA parks its partial in its own ring (all of its MMAs have completed
                        // and nothing is in flight into the ring any more), the cluster meets, the partials are summed in rank
                        // order and stored, and the cluster meets again before anyone's shared memory goes away.
                        float* park = (float*)ring + (size_t)cb * 128 + etid;
#pragma unroll
                        for (int j = 0; j < NC; ++j) park[(size_t)j * 128] = acc[j];
                        cluster_barrier();
                        if (NC * ksl <= 32) {
                            // few columns and few slices: CTA 0 adds the others' partials (all NC loads of a peer in flight
                            // together) and stores; measured ~1 us faster than spreading so little work over the cluster
                            if (krank == 0) {
                                for (int pr = 1; pr < ksl; ++pr) {
#pragma unroll
                                    for (int j = 0; j < NC; ++j) acc[j] += ld_cluster_f32(park + (size_t)j * 128, (uint32_t)pr);
                                }
                            }
                            cluster_barrier();
                            cluster_done = true;
                            do_store = krank == 0;
                        } else {
                        // The token columns are dealt in contiguous blocks to the CTAs of the cluster: each sums its block
                        // over all ranks (rank order: the same sum on every run) and stores it, so the remote reads of the
                        // reduce run on all CTAs at once.  Eight columns at a time: their loads from every rank are in
                        // flight together, then the eight stores.
                        const int cols_per = NC / ksl < 2 ? 2 : NC / ksl;   // (a SwiGLU pair stays in one CTA)
                        const int jbeg = krank * cols_per, jend = jbeg + cols_per < NC ? jbeg + cols_per : NC;
                        uint32_t rbase[8];
#pragma unroll
                        for (int pr = 0; pr < 8; ++pr)
                            asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(rbase[pr]) : "r"(smem_u32(park)), "r"(pr < ksl ? pr : 0));
                        const int row = rt * 128 + r;
                        for (int jc = jbeg; jc < jend; jc += 8) {
                            float sum[8];
#pragma unroll
                            for (int u = 0; u < 8; ++u) sum[u] = 0.f;
#pragma unroll
                            for (int pr = 0; pr < 8; ++pr) {
#pragma unroll
                                for (int u = 0; u < 8; ++u) {
                                    if (pr < ksl && jc + u < jend) {
                                        float v;
                                        asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(rbase[pr] + (uint32_t)(jc + u) * 512u) : "memory");
                                        sum[u] += v;
                                    }
                                }
                            }
                            if (a.swiglu) {
                                // as the single-CTA SwiGLU store below: lanes l and l^8 hold a gate row and its up row
                                bf16* ocol = (bf16*)a.out + rt * 64 + (r >> 4) * 8 + (r & 7);
                                const float L = a.swiglu_limit;
                                const bool is_gate = (r & 8) == 0;
#pragma unroll
                                for (int u = 0; u < 8; u += 2) {
                                    const float o0 = __shfl_xor_sync(0xffffffffu, sum[u], 8);
                                    const float o1 = __shfl_xor_sync(0xffffffffu, sum[u + 1], 8);
                                    const int col = jc + (is_gate ? u : u + 1);
                                    if (jc + u < jend && cb + col < cnt && row < a.n_rows) {
                                        float gt = bf16_round(is_gate ? sum[u] : o1), up = bf16_round(is_gate ? o0 : sum[u + 1]);
                                        if (L > 0.f) { up = fminf(fmaxf(up, -L), L); gt = fminf(gt, L); }
                                        ocol[(size_t)(cb + col) * a.ldo] = __float2bfloat16(gt / (1.0f + expf(-gt)) * up);
                                    }
                                }
                            } else {
#pragma unroll
                                for (int u = 0; u < 8; ++u) {
                                    const float v = sum[u] * a.alpha;
                                    const bool mine = jc + u < jend && cb + jc + u < cnt && row < a.n_rows;
                                    if (a.rope_cos) {
                                        const float pv = __shfl_xor_sync(0xffffffffu, v, 1);   // row ^ 1 is the neighbouring lane
                                        if (mine) dense_store_rope(a, cb + jc + u, row, v, pv);
                                    } else if (mine) {
                                        dense_store(a, cb + jc + u, row, v);
                                    }
                                }
                            }
                        }
                        cluster_barrier();
                        cluster_done = true;
                        do_store = false;   // stored above
                        }
                    } else if (!whole) {
                        const int slot = (q == beg / KT) ? 0 : 1;
                        float* pw = a.partial + ((size_t)(c * 2 + slot) * 64 + cb) * 128 + etid;
#pragma unroll
                        for (int j = 0; j < NC; ++j) __stcg(pw + (size_t)j * 128, acc[j]);
                        __threadfence();
                        named_bar_sync(1, EPI_BAR);
                        const long long tot = (long long)RT * KT;
                        const int first = (int)(((it0 + 1) * G - 1) / tot);
                        const int last = (int)(((it0 + KT) * G - 1) / tot);
                        if (etid == 0 && eg == 0) {
                            const int old = atomicAdd(a.counters + q, 1);
                            s_flag = (old == last - first);
                            if (old == last - first) a.counters[q] = 0;  // self-resetting for the next launch
                        }
                        named_bar_sync(1, EPI_BAR);
                        do_store = s_flag != 0;
                        named_bar_sync(1, EPI_BAR);
                        if (do_store) {
                            __threadfence();
#pragma unroll
                            for (int j = 0; j < NC; ++j) acc[j] = 0.f;
                            for (int cc = first; cc <= last; ++cc) {  // fixed order: independent of arrival order
                                const long long cbeg = (long long)cc * tot / G;
                                const int cslot = (q == cbeg / KT) ? 0 : 1;
                                const float* pr = a.partial + ((size_t)(cc * 2 + cslot) * 64 + cb) * 128 + etid;
#pragma unroll
                                for (int j = 0; j < NC; ++j) acc[j] += __ldcg(pr + (size_t)j * 128);
                            }
                        }
                    }
                    if (do_store) {
                        const int row = rt * 128 + r;
                        if (a.swiglu) {
                            // gate / up rows interleaved 8 + 8 per 16-row group: lanes l and l^8 exchange, as in the expert
                            // epilogue below, without a routing weight (the shared expert applies to every token)
                            bf16* ocol = (bf16*)a.out + rt * 64 + (r >> 4) * 8 + (r & 7);
                            const float L = a.swiglu_limit;
                            const bool is_gate = (r & 8) == 0;
#pragma unroll
                            for (int j = 0; j < NC; j += 2) {
                                const float o0 = __shfl_xor_sync(0xffffffffu, acc[j], 8);
                                const float o1 = __shfl_xor_sync(0xffffffffu, acc[j + 1], 8);
                                const int col = is_gate ? j : j + 1;
                                if (cb + col < cnt && row < a.n_rows) {
                                    float gt = bf16_round(is_gate ? acc[j] : o1), up = bf16_round(is_gate ? o0 : acc[j + 1]);
                                    if (L > 0.f) { up = fminf(fmaxf(up, -L), L); gt = fminf(gt, L); }
                                    ocol[(size_t)(cb + col) * a.ldo] = __float2bfloat16(gt / (1.0f + expf(-gt)) * up);
                                }
                            }
                        } else {
#pragma unroll
                            for (int j = 0; j < NC; ++j) {
                                const float v = acc[j] * a.alpha;
                                const bool mine = cb + j < cnt && row < a.n_rows;
                                if (a.rope_cos) {
                                    const float pv = __shfl_xor_sync(0xffffffffu, v, 1);   // row ^ 1 is the neighbouring lane
                                    if (mine) dense_store_rope(a, cb + j, row, v, pv);
                                } else if (mine) {
                                    dense_store(a, cb + j, row, v);
                                }
                            }
                        }
                    }
                } else if (EPI == EPI_W13) {
                    // lanes l and l^8 hold a gate row and its up row (rows 0..7 / 8..15 of every 16-row group);
                    // SwiGLU as crates/kernels/cu/gemv.cu:470-483: bf16 rounds, optional clamp, routing weight folded in
                    bf16* o = (bf16*)a.out;
                    const float L = a.swiglu_limit;
                    const bool is_gate = (r & 8) == 0;
                    bf16* ocol = o + rt * 64 + (r >> 4) * 8 + (r & 7);
                    // After the exchange both lanes of a pair hold (gate, up) of two token columns: the gate lane
                    // finishes column j, the up lane column j + 1, so every lane evaluates one SwiGLU per column pair.
#pragma unroll
                    for (int j = 0; j < NC; j += 2) {
                        const float o0 = __shfl_xor_sync(0xffffffffu, acc[j], 8);
                        const float o1 = __shfl_xor_sync(0xffffffffu, acc[j + 1], 8);
                        const int col = is_gate ? j : j + 1;
                        const float rw = __shfl_sync(0xffffffffu, rwreg[col >> 5], col & 31);
                        if (cb + col < cnt) {
                            const int row = xrow0 + cb + col;
                            float gt = bf16_round(is_gate ? acc[j] : o1), up = bf16_round(is_gate ? o0 : acc[j + 1]);
                            if (L > 0.f) { up = fminf(fmaxf(up, -L), L); gt = fminf(gt, L); }
                            const float val = gt / (1.0f + expf(-gt)) * up * rw;
                            ocol[(size_t)row * a.ldo] = __float2bfloat16(val);
                        }
                    }
                } else {
                    float* o = (float*)a.out;
                    const int col = rt * 128 + r;
#pragma unroll
                    for (int j = 0; j < NC; ++j)
                        if (cb + j < cnt && col < a.n_rows) o[(size_t)(xrow0 + cb + j) * a.ldo + col] = acc[j];
                }
            }
            if (item_end) {
#pragma unroll
                for (int j = 0; j < NC; ++j) acc[j] = 0.f;
                g0 = i + 1;
            }
            est += Cfg::STAGE;
            if (++es == S) { es = 0; est = ring; }
            if (++kt == KT) { kt = 0; ++q; fresh = true; }
        }
    }
    if (ksl > 1 && !cluster_done) {
        // warps that hold no partial sum still take part in the reduce's two cluster-wide barriers
        cluster_barrier();
        cluster_barrier();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    if (warp == 1) tmem_dealloc(tm, Cfg::TM_COLS);
}

}  // namespace dsuf
