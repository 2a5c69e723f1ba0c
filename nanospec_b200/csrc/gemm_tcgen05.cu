// bfloat16 matrix product on the 5th-generation tensor cores: out[M, N] = x[M, K] * w[N, K]^T.
//
// The product is computed transposed ("swap A/B"): the weight rows (output features) are the M
// side of tcgen05.mma (128 per block, one TMEM lane each) and the tokens are its N side (16 to
// 256 per block).  That keeps the tensor core's 128 lanes full for any number of tokens, so the
// same kernel streams weights for a decode step of a few tokens and tiles a prompt of thousands.
//
// One block = 6 warps with fixed roles:
//   warp 0, one lane: TMA producer.  Per 64-wide k block it waits for a free stage, arms the
//           stage's mbarrier with the byte count and issues two cp.async.bulk.tensor loads (weight
//           tile 128 x 64, token tile BN x 64) into 128-byte-swizzled shared memory.
//   warp 1, one lane: MMA issuer.  Waits for a full stage, issues four tcgen05.mma (k = 16 each)
//           with shared-memory descriptors, accumulating in TMEM, and commits to the stage's
//           "empty" mbarrier so the producer may refill it; after the last k block it commits to
//           the "accumulator ready" mbarrier.  Warp 1 also allocates and frees the TMEM columns.
//   warps 2-5: epilogue.  Each warp reads its 32 TMEM lanes with tcgen05.ld and stores
//           out[token, feature] (a warp writes 32 consecutive features of one token).
// Split-K: with `splits` in {2, 4, 8} the k blocks of one output tile are divided among the blocks
// of a thread-block cluster; each leaves its fp32 partial tile in its shared memory and, after a
// cluster barrier, adds one slice of the features from all blocks' shared memory in rank order.
// Gated mode (the feed-forward's packed projection): the weight rows alternate between 64 gate and
// 64 up features, so a block's tile holds both halves of 64 outputs and the epilogue writes
// silu(gate) * up - the activation costs no kernel and no trip through global memory.
// Two more epilogues let a decode step do without its norm kernels (64 tokens at most):
//   sink:  the output is a branch of the residual stream that an RMSNorm follows.  The block adds
//          its features to the fp32 residual, writes gain * residual in bf16 for the next product and
//          the sum of squares of its features per token; the norm's scale, one number per token, is
//          still missing from those activations.
//   rope:  the product is the packed q/k/v projection: the epilogue rotates q and k by the token's position
//          and writes k and v straight to the token's cache slot - no rotation kernel, and k and v never
//          travel through the projection's output buffer.
//   scale: the activations came from such a sink.  The epilogue adds up the partial sums of squares of
//          each token (in a fixed order), and multiplies the token's outputs by
//          rsqrt(sum / hidden + eps) - a product is linear in a per-token scale of its input.
//
// Every wait on an mbarrier is bounded (two seconds): when it runs out the thread records a code
// in *error_flag and the block winds down (copies in flight are awaited, again bounded, TMEM is
// freed).  The host reads the flag after the stream has been synchronised.
#include "tcgen05_utils.cuh"

namespace {

constexpr int BM = 128;            // features per block = UMMA M
constexpr int BK = 64;             // k per stage: 64 bf16 = one 128-byte swizzle row
constexpr int UMMA_K = 16;
constexpr int kThreads = 192;
constexpr int kMaxSplits = 8;

// What the epilogue does besides storing the product (all pointers null: nothing).
struct GemmEpilogue {
    int gated;                    // silu(gate) * up on alternating runs of 64 features
    // scale: out rows *= rsqrt(sum_p row_partials[token, p] / hidden + eps)
    const float* row_partials;    // [tokens, n_partials]
    int n_partials;
    float inv_hidden, eps;
    // sink: resid += product; sink_x = bf16(gain * resid); sink_partials[token, block] = sum of resid^2 over the block's features
    float* sink_resid;            // [tokens, sink_ld]
    const float* sink_gain;       // [features]
    __nv_bfloat16* sink_x;        // [tokens, sink_ld]
    float* sink_partials;         // [tokens, feature tiles * splits]
    int sink_ld;
    // rope: the product is an attention layer's packed [q | k | v] projection.  q and k are rotated by the
    // token's position (pairs (j, j + head_dim / 2)); q goes to `out`, k and v to the token's slot of the cache
    // [page, kv head, offset, head_dim].  Tiles of 128 features hold whole heads (head_dim 32, 64 or 128).
    const int* rope_positions;    // [tokens]; null: no rope epilogue
    const int* rope_token_req;    // [tokens], negative: a padding row
    const int* rope_block_table;  // [requests, rope_table_stride]
    const float* rope_inv_freq;   // [rope_pairs]
    __nv_bfloat16* rope_k_cache;
    __nv_bfloat16* rope_v_cache;
    int rope_table_stride, rope_page_size, rope_nq, rope_nkv, rope_head_dim, rope_pairs, rope_write_kv;
};

enum GemmError { kErrProducerWait = 1, kErrMmaWait = 2, kErrEpilogueWait = 3, kErrDrainWait = 4 };

template <int BN>
struct Cfg {
    // up to 64 tokens: stages sized so that two blocks share an SM (8 to 12 tiles in flight per SM)
    static constexpr int kStages = BN == 16 ? 6 : BN == 32 ? 5 : (BN == 64 ? 4 : (BN == 128 ? 6 : 4));
    static constexpr int kMinBlocks = BN <= 64 ? 2 : 1;
    static constexpr int kABytes = BM * BK * 2;
    static constexpr int kBBytes = BN * BK * 2;
    static constexpr int kStageBytes = kABytes + kBBytes;
    static constexpr int kTmemCols = BN < 32 ? 32 : BN;
    static constexpr size_t kSmemBytes = (size_t)kStages * kStageBytes + 1024 /* alignment slack */ + 256 /* barriers */;
};

// Instruction descriptor: D = fp32, A = B = bf16, both K-major, M = 128, N = BN.
template <int BN>
__device__ __forceinline__ constexpr uint32_t instr_desc() {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
}

__device__ __forceinline__ void tmem_ld_cols(uint32_t taddr, uint32_t (&r)[16]) { tmem_ld16(taddr, r); }
__device__ __forceinline__ void tmem_ld_cols(uint32_t taddr, uint32_t (&r)[32]) { tmem_ld32(taddr, r); }

__device__ __forceinline__ void store_out(float* p, float v) { *p = v; }
__device__ __forceinline__ void store_out(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }
// two neighbouring outputs at an address aligned for the pair
__device__ __forceinline__ void store_out2(float* p, float a, float b) { *reinterpret_cast<float2*>(p) = make_float2(a, b); }
__device__ __forceinline__ void store_out2(__nv_bfloat16* p, float a, float b) {
    *reinterpret_cast<__nv_bfloat162*>(p) = __floats2bfloat162_rn(a, b);
}
// four neighbouring outputs: one store where the address allows it
__device__ __forceinline__ void store_out4(float* p, const float4& v) {
    if ((reinterpret_cast<uintptr_t>(p) & 15) == 0) *reinterpret_cast<float4*>(p) = v;
    else { p[0] = v.x; p[1] = v.y; p[2] = v.z; p[3] = v.w; }
}
__device__ __forceinline__ void store_out4(__nv_bfloat16* p, const float4& v) {
    if ((reinterpret_cast<uintptr_t>(p) & 7) == 0) {
        const __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
        *reinterpret_cast<uint2*>(p) = make_uint2(*reinterpret_cast<const uint32_t*>(&lo), *reinterpret_cast<const uint32_t*>(&hi));
    } else {
        p[0] = __float2bfloat16_rn(v.x); p[1] = __float2bfloat16_rn(v.y);
        p[2] = __float2bfloat16_rn(v.z); p[3] = __float2bfloat16_rn(v.w);
    }
}

template <int BN, typename OutT>
__global__ void __launch_bounds__(kThreads, Cfg<BN>::kMinBlocks)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
               OutT* __restrict__ out, int ldo, int M_tok, int N_feat, int k_blocks, int splits, const GemmEpilogue ep,
               int* __restrict__ error_flag) {
    const int gated = ep.gated;
    const bool sink = ep.sink_resid != nullptr;
    const bool rope = ep.rope_positions != nullptr;
    // per-token scale (scale mode) and squares of the finished residual (sink mode); both modes are
    // offered for tiles of up to 64 tokens
    constexpr bool kNorm = BN <= 64;
    __shared__ float inv_s[kNorm ? BN : 1];
    using C = Cfg<BN>;
    extern __shared__ unsigned char smem_dyn[];
    const uint32_t base = (smem_u32(smem_dyn) + 1023u) & ~1023u;  // swizzled tiles need 1024-byte alignment
    const uint32_t bar_base = base + C::kStages * C::kStageBytes;
    // barriers: full[kStages], empty[kStages], accum, then the TMEM address holder
    auto full_bar = [&](int s) { return bar_base + 8u * s; };
    auto empty_bar = [&](int s) { return bar_base + 8u * (C::kStages + s); };
    const uint32_t accum_bar = bar_base + 8u * (2 * C::kStages);
    const uint32_t holder = accum_bar + 8u;
    __shared__ int failed;
    // after the last MMA the pipeline stages are free: the split-K partial tile is staged there
    float* stage_f32 = reinterpret_cast<float*>(smem_dyn + (base - smem_u32(smem_dyn)));
    float* sq_s = stage_f32 + BN * BM;  // sink mode: [BN][BM + 1] squares, behind the partial tile

    ns_pdl_launch_dependents();  // the next kernel may be scheduled; it waits for this one before it reads
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n0 = blockIdx.x * BM;      // first feature of the tile
    const int tok0 = blockIdx.y * BN;    // first token of the tile
    const int split = blockIdx.z;
    // this block's k blocks
    const int per = k_blocks / splits, rem = k_blocks % splits;
    const int kb_begin = split * per + min(split, rem);
    const int kb_count = per + (split < rem ? 1 : 0);

    // rope mode: what a thread needs for its first (token, four pairs) of the reduction below, fetched while the product runs
    float rope_sin0[4] = {0.f, 0.f, 0.f, 0.f}, rope_cos0[4] = {1.f, 1.f, 1.f, 1.f};
    int rope_req0 = -1, rope_pos0 = 0, rope_page0 = 0;
    if (threadIdx.x == 0) {
        failed = 0;
        for (int s = 0; s < C::kStages; ++s) {
            mbar_init(full_bar(s), 1);
            mbar_init(empty_bar(s), 1);
        }
        mbar_init(accum_bar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) tmem_alloc(holder, C::kTmemCols);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    uint32_t tmem_base;
    asm volatile("ld.shared.b32 %0, [%1];" : "=r"(tmem_base) : "r"(holder));

    if (warp == 0) {
        // ---------------- TMA producer: the warp runs the loop converged, one elected lane issues ----------------
        // The weights do not depend on the previous kernel: their first tiles are requested before
        // this kernel waits for it, so they stream in while the predecessor is still running.  The
        // token tiles of those stages follow after the wait (each stage's barrier counts both).
        int issued = 0;
        bool ok = true;
        const int early = min(kb_count, C::kStages);
        if (elect_one()) {
            for (int i = 0; i < early; ++i) {
                mbar_expect_tx(full_bar(i), C::kStageBytes);
                tma_load_2d(base + i * C::kStageBytes, &map_w, (kb_begin + i) * BK, n0, full_bar(i));
            }
        }
        ns_pdl_wait();
        if (elect_one()) {
            for (int i = 0; i < early; ++i)
                tma_load_2d(base + i * C::kStageBytes + C::kABytes, &map_x, (kb_begin + i) * BK, tok0, full_bar(i));
        }
        issued = early;
        for (int i = early; i < kb_count; ++i) {
            const int s = i % C::kStages;
            const uint32_t ph = (uint32_t)(i / C::kStages) & 1u;
            if (!mbar_wait_warp(empty_bar(s), ph ^ 1u)) {
                ok = false;
                if (lane == 0) atomicExch(error_flag, kErrProducerWait);
                break;
            }
            if (elect_one()) {
                mbar_expect_tx(full_bar(s), C::kStageBytes);
                const uint32_t a = base + s * C::kStageBytes;
                tma_load_2d(a, &map_w, (kb_begin + i) * BK, n0, full_bar(s));
                tma_load_2d(a + C::kABytes, &map_x, (kb_begin + i) * BK, tok0, full_bar(s));
            }
            ++issued;
        }
        if (!ok) {
            // wait, bounded, for the copies that are still in flight before the block may exit
            if (lane == 0) failed = 1;
            for (int i = max(0, issued - C::kStages); i < issued; ++i)
                if (!mbar_wait_warp(full_bar(i % C::kStages), (uint32_t)(i / C::kStages) & 1u)) {
                    if (lane == 0) atomicExch(error_flag, kErrDrainWait);
                    break;
                }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer: the warp runs the loop converged, one elected lane issues ----------------
        constexpr uint32_t idesc = instr_desc<BN>();
        for (int i = 0; i < kb_count; ++i) {
            const int s = i % C::kStages;
            const uint32_t ph = (uint32_t)(i / C::kStages) & 1u;
            if (!mbar_wait_warp(full_bar(s), ph)) {
                if (lane == 0) { failed = 1; atomicExch(error_flag, kErrMmaWait); }
                break;
            }
            tc_fence_after();
            const uint32_t a = base + s * C::kStageBytes;
            const uint32_t b = a + C::kABytes;
            if (elect_one()) {
#pragma unroll
                for (int k = 0; k < BK / UMMA_K; ++k)
                    umma_bf16(tmem_base, smem_desc(a + k * UMMA_K * 2), smem_desc(b + k * UMMA_K * 2), idesc,
                              (i > 0 || k > 0) ? 1u : 0u);
                umma_commit(empty_bar(s));  // the stage is free once these MMAs have read it
            }
        }
        if (elect_one()) umma_commit(accum_bar);  // the accumulator is complete once every MMA above has finished
    } else if (warp >= 2) {
        // ---------------- epilogue ----------------
        ns_pdl_wait();           // before anything is written that the previous kernel may still read
        const int q = warp & 3;  // the TMEM lane quarter this warp may read
        const int f = n0 + q * 32 + lane;
        if (kNorm) {
            // While the products run: each token's scale.  A warp takes four tokens at a time, a lane every 32nd
            // partial sum of each (the loads of all four are requested before the first is used), then the lanes'
            // sums are added in a fixed tree: the same value in every block, whatever the timing.
            for (int t0 = warp - 2; t0 < BN; t0 += 16) {
                float acc[4] = {0.f, 0.f, 0.f, 0.f};
                if (ep.row_partials) {
                    for (int i0 = 0; i0 < ep.n_partials; i0 += 256) {
                        float v[4][8];
#pragma unroll
                        for (int u = 0; u < 4; ++u) {
                            const int t = t0 + 4 * u;
                            const bool live = t < BN && tok0 + t < M_tok;
                            const float* p = ep.row_partials + (size_t)(live ? tok0 + t : 0) * ep.n_partials;
#pragma unroll
                            for (int k = 0; k < 8; ++k) {
                                const int i = i0 + lane + 32 * k;
                                v[u][k] = live && i < ep.n_partials ? __ldg(p + i) : 0.f;
                            }
                        }
#pragma unroll
                        for (int u = 0; u < 4; ++u)
#pragma unroll
                            for (int k = 0; k < 8; ++k) acc[u] += v[u][k];
                    }
                }
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const int t = t0 + 4 * u;
                    if (t >= BN) break;  // uniform across the warp
                    float inv = 1.f;
                    if (ep.row_partials && tok0 + t < M_tok) inv = rsqrtf(ns_warp_sum(acc[u]) * ep.inv_hidden + ep.eps);
                    if (lane == 0) inv_s[t] = inv;
                }
            }
            asm volatile("bar.sync 1, 128;" ::: "memory");  // the four epilogue warps
        }
        if (kNorm && rope) {
            // this thread's first (token, four pairs) of the reduction below: the token's request, position, cache page
            // and angles do not wait for the product
            const int half = ep.rope_head_dim / 2;
            const int groups = ((BM / 2) / splits) >> 2;
            const int e = (int)threadIdx.x - 64;
            const int tok_n = min(BN, M_tok - tok0);
            if (e < tok_n * groups) {
                const int j = e / groups, pid = split * (groups << 2) + 4 * (e - j * groups);
                const int head_local = pid / half, p = pid - head_local * half;
                const int gh = n0 / ep.rope_head_dim + head_local;
                rope_req0 = ep.rope_token_req[tok0 + j];
                rope_pos0 = ep.rope_positions[tok0 + j];
                if (rope_req0 >= 0) {
                    if (gh >= ep.rope_nq && ep.rope_write_kv)
                        rope_page0 = ep.rope_block_table[(size_t)rope_req0 * ep.rope_table_stride + rope_pos0 / ep.rope_page_size];
                    if (gh < ep.rope_nq + ep.rope_nkv) {
#pragma unroll
                        for (int c = 0; c < 4; ++c)
                            if (p + c < ep.rope_pairs) sincosf((float)rope_pos0 * ep.rope_inv_freq[p + c], &rope_sin0[c], &rope_cos0[c]);
                    }
                }
            }
        }
        const bool ok = mbar_wait_warp(accum_bar, 0);
        if (!ok) {
            if (lane == 0) { failed = 1; atomicExch(error_flag, kErrEpilogueWait); }
        } else {
            tc_fence_after();
            const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16);
            // 16 or 32 tokens' columns per wait (a lane holds one feature of each)
            constexpr int CH = BN >= 32 ? 32 : 16;
#pragma unroll 1
            for (int c0 = 0; c0 < BN; c0 += CH) {
                if (tok0 + c0 >= M_tok) break;  // uniform across the warp
                uint32_t r[CH];
                tmem_ld_cols(taddr + c0, r);
                tmem_ld_wait();
                if (f < N_feat) {
#pragma unroll
                    for (int j = 0; j < CH; ++j) {
                        const int tok = tok0 + c0 + j;
                        if (tok < M_tok) {
                            const float v = __uint_as_float(r[j]);
                            if (splits == 1 && !gated && !sink && !rope) store_out(out + (size_t)tok * ldo + f, kNorm ? v * inv_s[c0 + j] : v);
                            else stage_f32[(c0 + j) * BM + q * 32 + lane] = v;  // this block's partial tile, [token][feature]
                        }
                    }
                }
            }
        }
    }

    // ---------------- wind down: free TMEM; with split-K the blocks of the cluster add their tiles ----------------
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, C::kTmemCols);
    }
    if (splits == 1 && !gated && !sink && !rope) return;

    // The `splits` blocks of one output tile form a thread-block cluster.  Each has left its fp32
    // partial tile in its own shared memory; after a cluster barrier every block adds, in rank
    // order, one slice of the features from all the blocks' shared memory (distributed shared
    // memory) and writes that slice of the result.  Nothing goes through global memory, and the
    // sum does not depend on timing.  Blocks that gave up still take part in both barriers.
    if (splits > 1) cluster_sync();
    const uint32_t stage_addr = smem_u32(stage_f32);
    // element idx of the partial tile of block s (a block without a cluster reads its own)
    auto partial = [&](int idx, int s) {
        return splits == 1 ? stage_f32[idx] : ld_cluster_f32(stage_addr + 4u * (uint32_t)idx, (uint32_t)s);
    };
    // four neighbouring elements (idx a multiple of four)
    auto partial4 = [&](int idx, int s) {
        return splits == 1 ? *reinterpret_cast<const float4*>(stage_f32 + idx)
                           : ld_cluster_f32x4(stage_addr + 4u * (uint32_t)idx, (uint32_t)s);
    };
    // The reductions below take four neighbouring features per thread and turn, and ask for everything a turn
    // needs from global memory before they ask for the partial tiles: a turn costs one round trip, and a tile of
    // 64 tokens has few turns per thread.
    if (!failed) {
        const int tok_n = min(BN, M_tok - tok0);
        if (kNorm && rope) {
            // Pairs (j, j + head_dim / 2) of a head are rotated together: this block finishes 64 / splits pairs
            // per token, both members of each.  The four epilogue warps do it (they hold what their first turn needs).
            const int D = ep.rope_head_dim, half = D / 2;
            const int groups = ((BM / 2) / splits) >> 2;                 // runs of four pairs per token: a power of two
            const int group_shift = 31 - __clz(groups);
            for (int e = (int)threadIdx.x - 64; e >= 0 && e < tok_n * groups; e += 128) {
                const bool first = e == (int)threadIdx.x - 64;
                const int j = e >> group_shift, pid = split * (groups << 2) + 4 * (e & (groups - 1));
                const int head_local = pid / half, p = pid - head_local * half;
                const int lo = head_local * D + p, hi = lo + half;       // features within the tile
                const int tok = tok0 + j;
                const int req = first ? rope_req0 : ep.rope_token_req[tok];
                if (req < 0 || n0 + hi >= N_feat) continue;
                const int pos = first ? rope_pos0 : ep.rope_positions[tok];
                const int gh = n0 / D + head_local;                     // head among [q | k | v]
                const bool is_q = gh < ep.rope_nq, rotated = gh < ep.rope_nq + ep.rope_nkv;
                int page = rope_page0;
                if (!first && !is_q && ep.rope_write_kv)
                    page = ep.rope_block_table[(size_t)req * ep.rope_table_stride + pos / ep.rope_page_size];
                float4 a[kMaxSplits], b[kMaxSplits];
#pragma unroll
                for (int s2 = 0; s2 < kMaxSplits; ++s2) {
                    a[s2] = s2 < splits ? partial4(j * BM + lo, s2) : make_float4(0.f, 0.f, 0.f, 0.f);
                    b[s2] = s2 < splits ? partial4(j * BM + hi, s2) : make_float4(0.f, 0.f, 0.f, 0.f);
                }
                float x1[4] = {0.f, 0.f, 0.f, 0.f}, x2[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                for (int s2 = 0; s2 < kMaxSplits; ++s2) {
                    x1[0] += a[s2].x; x1[1] += a[s2].y; x1[2] += a[s2].z; x1[3] += a[s2].w;
                    x2[0] += b[s2].x; x2[1] += b[s2].y; x2[2] += b[s2].z; x2[3] += b[s2].w;
                }
                float o1[4], o2[4];
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    x1[c] *= inv_s[j];
                    x2[c] *= inv_s[j];
                    o1[c] = x1[c];
                    o2[c] = x2[c];
                    if (rotated && p + c < ep.rope_pairs) {
                        float sn = rope_sin0[c], cs = rope_cos0[c];
                        if (!first) sincosf((float)pos * ep.rope_inv_freq[p + c], &sn, &cs);
                        o1[c] = __fmaf_rn(x1[c], cs, -__fmul_rn(x2[c], sn));
                        o2[c] = __fmaf_rn(x2[c], cs, __fmul_rn(x1[c], sn));
                    }
                }
                const float4 w1 = make_float4(o1[0], o1[1], o1[2], o1[3]), w2 = make_float4(o2[0], o2[1], o2[2], o2[3]);
                if (is_q) {
                    OutT* dst = out + (size_t)tok * ldo + (size_t)gh * D + p;
                    store_out4(dst, w1);
                    store_out4(dst + half, w2);
                } else if (ep.rope_write_kv) {
                    const bool is_v = !rotated;
                    const int hk = gh - ep.rope_nq - (is_v ? ep.rope_nkv : 0);
                    __nv_bfloat16* dst = (is_v ? ep.rope_v_cache : ep.rope_k_cache) +
                        (((size_t)page * ep.rope_nkv + hk) * ep.rope_page_size + pos % ep.rope_page_size) * D + p;
                    store_out4(dst, w1);
                    store_out4(dst + half, w2);
                }
            }
        } else if (!gated) {
            const int slice = BM / splits;             // features this block reduces: a power of two, 16 at least
            const int i0 = split * slice;
            const int groups = slice >> 2;             // runs of four features per token
            const int group_shift = 31 - __clz(groups);
            for (int e = threadIdx.x; e < tok_n * groups; e += kThreads) {
                const int j = e >> group_shift, i = i0 + 4 * (e & (groups - 1));
                if (n0 + i >= N_feat) continue;
                float4 res = make_float4(0.f, 0.f, 0.f, 0.f);
                float gain[4] = {0.f, 0.f, 0.f, 0.f};
                const size_t so = (size_t)(tok0 + j) * ep.sink_ld + n0 + i;
                if (kNorm && sink) {  // a sink's width is whole tiles, its rows are 16-byte aligned (checked by the host)
                    res = *reinterpret_cast<const float4*>(ep.sink_resid + so);
#pragma unroll
                    for (int c = 0; c < 4; ++c) gain[c] = __ldg(ep.sink_gain + n0 + i + c);
                }
                float4 v[kMaxSplits];
#pragma unroll
                for (int s = 0; s < kMaxSplits; ++s) v[s] = s < splits ? partial4(j * BM + i, s) : make_float4(0.f, 0.f, 0.f, 0.f);
                float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                for (int s = 0; s < kMaxSplits; ++s) { acc.x += v[s].x; acc.y += v[s].y; acc.z += v[s].z; acc.w += v[s].w; }
                if (kNorm) {
                    const float inv = inv_s[j];
                    acc.x *= inv; acc.y *= inv; acc.z *= inv; acc.w *= inv;
                }
                if (kNorm && sink) {
                    res.x += acc.x; res.y += acc.y; res.z += acc.z; res.w += acc.w;
                    *reinterpret_cast<float4*>(ep.sink_resid + so) = res;
                    store_out4(ep.sink_x + so, make_float4(res.x * gain[0], res.y * gain[1], res.z * gain[2], res.w * gain[3]));
                    float* sq = sq_s + j * (BM + 1) + (i - i0);
                    sq[0] = res.x * res.x; sq[1] = res.y * res.y; sq[2] = res.z * res.z; sq[3] = res.w * res.w;
                } else {
                    OutT* dst = out + (size_t)(tok0 + j) * ldo + n0 + i;
                    if (n0 + i + 3 < N_feat) {
                        store_out4(dst, acc);
                    } else {
                        store_out(dst, acc.x);
                        if (n0 + i + 1 < N_feat) store_out(dst + 1, acc.y);
                        if (n0 + i + 2 < N_feat) store_out(dst + 2, acc.z);
                    }
                }
            }
            if (kNorm && sink) {
                // the block's share of each token's sum of squares, added in feature order
                __syncthreads();
                if ((int)threadIdx.x < tok_n) {
                    float t = 0.f;
                    for (int k = 0; k < slice; ++k) t += sq_s[threadIdx.x * (BM + 1) + k];
                    ep.sink_partials[(size_t)(tok0 + threadIdx.x) * (gridDim.x * splits) + blockIdx.x * splits + split] = t;
                }
            }
        } else {
            // features 0..63 of the tile are gates, 64..127 the matching ups: this block finishes
            // 64 / splits outputs per token
            const int slice = (BM / 2) / splits;        // a power of two, 8 at least
            const int i0 = split * slice;
            const int o0 = n0 / 2;                      // first output feature of the tile
            const int half_shift = 31 - __clz(slice) - 1;
            // two neighbouring outputs per thread and turn: 8-byte reads of the partial tiles, one 4-byte store
            for (int e = threadIdx.x; e < tok_n * (slice / 2); e += kThreads) {
                const int j = e >> half_shift, i = i0 + 2 * (e & (slice / 2 - 1));
                if (2 * (o0 + i) >= N_feat) continue;
                float2 gs = make_float2(0.f, 0.f), us = make_float2(0.f, 0.f);
                if (splits == 1) {
                    gs = *reinterpret_cast<const float2*>(stage_f32 + j * BM + i);
                    us = *reinterpret_cast<const float2*>(stage_f32 + j * BM + BM / 2 + i);
                } else {
                    float2 g[kMaxSplits], u[kMaxSplits];
#pragma unroll
                    for (int s = 0; s < kMaxSplits; ++s) {
                        g[s] = s < splits ? make_float2(partial(j * BM + i, s), partial(j * BM + i + 1, s)) : make_float2(0.f, 0.f);
                        u[s] = s < splits ? make_float2(partial(j * BM + BM / 2 + i, s), partial(j * BM + BM / 2 + i + 1, s))
                                          : make_float2(0.f, 0.f);
                    }
#pragma unroll
                    for (int s = 0; s < kMaxSplits; ++s) {
                        gs.x += g[s].x; gs.y += g[s].y;
                        us.x += u[s].x; us.y += u[s].y;
                    }
                }
                if (kNorm) {
                    const float inv = inv_s[j];
                    gs.x *= inv; gs.y *= inv; us.x *= inv; us.y *= inv;
                }
                // silu(gate) * up; the hardware exponential and division (about 2 ulp in float) are far below the
                // rounding of the result
                const float r0 = __fdividef(gs.x, 1.f + __expf(-gs.x)) * us.x;
                const float r1 = __fdividef(gs.y, 1.f + __expf(-gs.y)) * us.y;
                OutT* dst = out + (size_t)(tok0 + j) * ldo + o0 + i;
                if (2 * (o0 + i + 1) < N_feat && (reinterpret_cast<uintptr_t>(dst) % (2 * sizeof(OutT))) == 0) {
                    store_out2(dst, r0, r1);
                } else {
                    store_out(dst, r0);
                    if (2 * (o0 + i + 1) < N_feat) store_out(dst + 1, r1);
                }
            }
        }
    }
    if (splits > 1) cluster_sync();  // no block may exit while another still reads its shared memory
}

// ---- host side ---------------------------------------------------------------------------------
template <int BN, typename OutT>
int launch_tc(const CUtensorMap& mw, const CUtensorMap& mx, void* out, int ldo, int M_tok, int N_feat, int k_blocks,
              int splits, const GemmEpilogue& ep, int* error_flag, cudaStream_t stream) {
    using C = Cfg<BN>;
    static bool configured = false;
    if (!configured) {
        NS_CUDA(cudaFuncSetAttribute(gemm_tc_kernel<BN, OutT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)C::kSmemBytes));
        configured = true;
    }
    dim3 grid((N_feat + BM - 1) / BM, (M_tok + BN - 1) / BN, splits);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = C::kSmemBytes;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    int n_attr = 0;
    if (ns_pdl_enabled) {
        attr[n_attr].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[n_attr].val.programmaticStreamSerializationAllowed = 1;
        ++n_attr;
    }
    if (splits > 1) {  // the blocks that share an output tile form a cluster along z
        attr[n_attr].id = cudaLaunchAttributeClusterDimension;
        attr[n_attr].val.clusterDim.x = 1;
        attr[n_attr].val.clusterDim.y = 1;
        attr[n_attr].val.clusterDim.z = splits;
        ++n_attr;
    }
    cfg.attrs = attr;
    cfg.numAttrs = n_attr;
    (void)cudaLaunchKernelEx(&cfg, gemm_tc_kernel<BN, OutT>, mw, mx, (OutT*)out, ldo, M_tok, N_feat, k_blocks, splits,
                             ep, error_flag);
    NS_CHECK_LAUNCH("ns_gemm_bf16_tc");
    return NS_OK;
}

}  // namespace

// Tokens per block the kernel would use for M_tok tokens, and the features per block.
NS_API int ns_gemm_bf16_tc_tile(int M_tok, int* tokens_per_block, int* features_per_block) {
    *tokens_per_block = M_tok <= 16 ? 16 : M_tok <= 32 ? 32 : M_tok <= 64 ? 64 : M_tok <= 128 ? 128 : 256;
    *features_per_block = BM;
    return NS_OK;
}

// out[M_tok, N_feat] (bf16 when out_f32 == 0, float otherwise, row stride ldo) =
//     x[M_tok, K] (bf16, row stride ldx) * w[N_feat, K]^T (bf16, row stride ldw).
// K, ldx and ldw must be multiples of 8 and the pointers 16-byte aligned (TMA); otherwise the call is
// refused with NS_ERR_UNSUPPORTED.  splits is 1, 2, 4 or 8 (blocks of a cluster that share the k range).
// `error_flag` is a device int that a timed-out wait sets.
static int gemm_tc_host(const void* x, const void* w, void* out, int M_tok, int N_feat, int K, int ldx, int ldw, int ldo,
                        int out_f32, int splits, const GemmEpilogue& ep, int* error_flag, cudaStream_t stream) {
    const int gated = ep.gated;
    if (M_tok <= 0 || N_feat <= 0) return NS_OK;
    if (K <= 0 || K % 8 || ldx % 8 || ldw % 8 || ((uintptr_t)x | (uintptr_t)w) % 16)
        NS_FAIL(NS_ERR_UNSUPPORTED, "ns_gemm_bf16_tc: K=%d ldx=%d ldw=%d must be multiples of 8 and operands 16-byte aligned", K, ldx, ldw);
    if (gated && N_feat % BM)
        NS_FAIL(NS_ERR_UNSUPPORTED, "ns_gemm_bf16_tc_gated: %d packed features are no multiple of %d", N_feat, BM);
    const int k_blocks = (K + BK - 1) / BK;
    if (splits < 1 || splits > k_blocks || splits > kMaxSplits || (splits & (splits - 1)))
        NS_FAIL(NS_ERR_ARGUMENT, "ns_gemm_bf16_tc: splits=%d with %d k blocks (1, 2, 4 or 8, at most the k blocks)", splits, k_blocks);
    if (!error_flag) NS_FAIL(NS_ERR_ARGUMENT, "ns_gemm_bf16_tc: no error flag");
    int bn, bm;
    ns_gemm_bf16_tc_tile(M_tok, &bn, &bm);
    if ((ep.row_partials || ep.sink_resid) && bn > 64)
        NS_FAIL(NS_ERR_UNSUPPORTED, "ns_gemm_bf16_tc: the norm epilogues take 64 tokens at most, not %d", M_tok);
    if (ep.sink_resid && (N_feat % BM || gated || !ep.sink_gain || !ep.sink_x || !ep.sink_partials))
        NS_FAIL(NS_ERR_UNSUPPORTED, "ns_gemm_bf16_tc: a sink needs %d features to be a multiple of %d, and all its tensors", N_feat, BM);
    if (ep.sink_resid && (ep.sink_ld % 4 || (uintptr_t)ep.sink_resid % 16))
        NS_FAIL(NS_ERR_UNSUPPORTED, "ns_gemm_bf16_tc: a sink's residual rows must be 16-byte aligned (row stride %d floats)", ep.sink_ld);
    if (ep.row_partials && ep.n_partials < 1) NS_FAIL(NS_ERR_ARGUMENT, "ns_gemm_bf16_tc: n_partials=%d", ep.n_partials);
    if (ep.rope_positions) {
        const int D = ep.rope_head_dim;
        if (bn > 64 || gated || ep.sink_resid || out_f32 || (D != 32 && D != 64 && D != 128) || ep.rope_pairs > D / 2 ||
            N_feat != (ep.rope_nq + 2 * ep.rope_nkv) * D || N_feat % BM || !ep.rope_token_req || !ep.rope_inv_freq ||
            (ep.rope_write_kv && (!ep.rope_block_table || !ep.rope_k_cache || !ep.rope_v_cache || ep.rope_page_size < 1)))
            NS_FAIL(NS_ERR_UNSUPPORTED, "ns_gemm_bf16_tc_rope: at most 64 tokens, head_dim 32, 64 or 128 (not %d), %d features in whole tiles of %d, bf16 output", D, N_feat, BM);
    }
    if ((M_tok + bn - 1) / bn > 65535) NS_FAIL(NS_ERR_UNSUPPORTED, "ns_gemm_bf16_tc: too many token tiles");
    CUtensorMap mw, mx;
    int rc = ns_make_map_bf16(&mw, w, N_feat, K, ldw, BM, "ns_gemm_bf16_tc");
    if (rc) return rc;
    rc = ns_make_map_bf16(&mx, x, M_tok, K, ldx, bn, "ns_gemm_bf16_tc");
    if (rc) return rc;
#define NS_TC_CASE(BNN)                                                                                                 \
    case BNN:                                                                                                           \
        return out_f32 ? launch_tc<BNN, float>(mw, mx, out, ldo, M_tok, N_feat, k_blocks, splits, ep, error_flag,       \
                                               stream)                                                                  \
                       : launch_tc<BNN, __nv_bfloat16>(mw, mx, out, ldo, M_tok, N_feat, k_blocks, splits, ep,           \
                                                       error_flag, stream);
    switch (bn) {
        NS_TC_CASE(16) NS_TC_CASE(32) NS_TC_CASE(64) NS_TC_CASE(128) NS_TC_CASE(256)
    }
#undef NS_TC_CASE
    NS_FAIL(NS_ERR_UNSUPPORTED, "ns_gemm_bf16_tc: tile of %d tokens", bn);
}

NS_API int ns_gemm_bf16_tc(const void* x, const void* w, void* out, int M_tok, int N_feat, int K, int ldx, int ldw,
                           int ldo, int out_f32, int splits, int* error_flag, cudaStream_t stream) {
    GemmEpilogue ep = {};
    return gemm_tc_host(x, w, out, M_tok, N_feat, K, ldx, ldw, ldo, out_f32, splits, ep, error_flag, stream);
}

// The gated feed-forward's first half in one kernel: w[N_feat, K] holds, for every run of 64 outputs, 64 gate
// rows followed by the 64 matching up rows (N_feat a multiple of 128);
// out[M_tok, N_feat / 2] = silu(x * gate^T) * (x * up^T), the sums and the activation in fp32.
NS_API int ns_gemm_bf16_tc_gated(const void* x, const void* w, void* out, int M_tok, int N_feat, int K, int ldx, int ldw,
                                 int ldo, int out_f32, int splits, int* error_flag, cudaStream_t stream) {
    GemmEpilogue ep = {};
    ep.gated = 1;
    return gemm_tc_host(x, w, out, M_tok, N_feat, K, ldx, ldw, ldo, out_f32, splits, ep, error_flag, stream);
}

// The same products with the norm epilogues (64 tokens at most).
//   row_partials [M_tok, n_partials] (or null): every output row is multiplied by
//       rsqrt(sum of the row's partials / hidden + eps) - the activations x were left unscaled by a sink;
//   sink_resid [M_tok, sink_ld] (or null; not with gated): the product is added to it, sink_x [M_tok, sink_ld] gets
//       bf16(sink_gain * resid) and sink_partials [M_tok, n_sink_partials] the sums of squares per block, where
//       n_sink_partials = (N_feat / 128) * splits; `out` is not written.
NS_API int ns_gemm_bf16_tc_norm(const void* x, const void* w, void* out, int M_tok, int N_feat, int K, int ldx, int ldw,
                                int ldo, int out_f32, int splits, int gated, const float* row_partials, int n_partials,
                                int hidden, float eps, float* sink_resid, const float* sink_gain, void* sink_x,
                                float* sink_partials, int sink_ld, int* error_flag, cudaStream_t stream) {
    GemmEpilogue ep = {};
    ep.gated = gated;
    ep.row_partials = row_partials;
    ep.n_partials = n_partials;
    ep.inv_hidden = hidden > 0 ? 1.f / (float)hidden : 0.f;
    ep.eps = eps;
    ep.sink_resid = sink_resid;
    ep.sink_gain = sink_gain;
    ep.sink_x = (__nv_bfloat16*)sink_x;
    ep.sink_partials = sink_partials;
    ep.sink_ld = sink_ld;
    return gemm_tc_host(x, w, out, M_tok, N_feat, K, ldx, ldw, ldo, out_f32, splits, ep, error_flag, stream);
}

// The packed q/k/v projection of an attention layer with the rotation and the cache write in its epilogue (64
// tokens at most; head_dim 32, 64 or 128; (nq + 2 nkv) * head_dim features in whole tiles of 128).  out [M_tok, ldo]
// receives the rotated q at columns 0 .. nq * head_dim (its k and v columns are not written); k (rotated) and v go to
// cache[page, kv head, offset, :] with page = block_table[token_req[n], positions[n] / page_size] when write_kv is
// set.  row_partials as in ns_gemm_bf16_tc_norm (or null).
NS_API int ns_gemm_bf16_tc_rope(const void* x, const void* w, void* out, int M_tok, int N_feat, int K, int ldx, int ldw,
                                int ldo, int splits, const float* row_partials, int n_partials, int hidden, float eps,
                                const int* positions, const int* token_req, const int* block_table, int table_stride,
                                const float* inv_freq, void* k_cache, void* v_cache, int page_size, int nq, int nkv,
                                int head_dim, int rot_pairs, int write_kv, int* error_flag, cudaStream_t stream) {
    GemmEpilogue ep = {};
    ep.row_partials = row_partials;
    ep.n_partials = n_partials;
    ep.inv_hidden = hidden > 0 ? 1.f / (float)hidden : 0.f;
    ep.eps = eps;
    ep.rope_positions = positions;
    ep.rope_token_req = token_req;
    ep.rope_block_table = block_table;
    ep.rope_table_stride = table_stride;
    ep.rope_inv_freq = inv_freq;
    ep.rope_k_cache = (__nv_bfloat16*)k_cache;
    ep.rope_v_cache = (__nv_bfloat16*)v_cache;
    ep.rope_page_size = page_size;
    ep.rope_nq = nq;
    ep.rope_nkv = nkv;
    ep.rope_head_dim = head_dim;
    ep.rope_pairs = rot_pairs;
    ep.rope_write_kv = write_kv;
    if (!positions) NS_FAIL(NS_ERR_ARGUMENT, "ns_gemm_bf16_tc_rope: no positions");
    return gemm_tc_host(x, w, out, M_tok, N_feat, K, ldx, ldw, ldo, 0, splits, ep, error_flag, stream);
}
