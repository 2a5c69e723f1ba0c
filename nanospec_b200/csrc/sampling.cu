// Token choice from fp32 logits: a first kernel with 16 blocks per row reduces the row's maximum, argmax and
// sum of exponentials; a second with one block per row finds the thresholds and draws.
//
// Follows the reference's pure functions (spec/sampling.py:24-42, engine/engine.py:385-402):
//   temperature == 0 : the argmax of the raw logits (lowest index on a tie);
//   otherwise        : z / temperature, optional top-k / top-p (tokens in descending order are
//                      kept while the mass before them is <= top_p and their rank is < top_k),
//                      log-softmax over the kept tokens, and an inverse-CDF draw in vocabulary
//                      order with the uniform u: the first token whose inclusive cumulative
//                      probability exceeds u * total, clamped to the last token.
// Also returned: the token's log-probability under the raw logits at temperature 1, and under
// the processed distribution it was drawn from (0 for greedy rows).
// Tie rule for the nucleus: tokens with equal logits are kept or dropped together by top-p;
// at the top-k boundary equal logits are taken in order of their index.  The two thresholds are found without a
// sort, a byte of the ordering key at a time (radix_threshold: four passes over the row each).
#include "common.cuh"

namespace {

constexpr int kThreads = 1024;

__device__ __forceinline__ unsigned order_key(float z) {
    const unsigned b = __float_as_uint(z);
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

struct RowArgs {
    const float* z;
    int vocab;
};

// The smallest key t such that measure(keys > t) <= target - the lowest key that is still kept - without a sort.
// The measure is a count (top-k) or the mass exp(v - max_s) in fixed point (top-p: steps of 2^-40, so that sums do not
// depend on the order of the atomics); for the mass the target is `fraction` of the row's total.
//   pass 1  every value goes into one of 256 bins of an eighth of a nat below the row's maximum (each warp into bins
//           of its own in shared memory, added in a fixed order afterwards; what lies 32 nats or more below goes to
//           the last bin through registers).  A scan from the top finds the bin that holds the threshold.
//   pass 2  the keys of that bin are collected in shared memory,
//   then    the threshold is found among them a byte of the key at a time (four rounds over the list).
// If the bin is the last one or holds more keys than the list, the bytes are found by passes over the row instead.
// *above = measure(keys > t).
constexpr int kBins = 256;
constexpr float kMassOneF = 1099511627776.f;  // 2^40
constexpr int kListCap = (kThreads / 32) * kBins * 2;  // u32 keys in the space of the warps' bins

__device__ __forceinline__ float key_value(unsigned key) {
    return __uint_as_float((key & 0x80000000u) ? (key & 0x7fffffffu) : ~key);
}
__device__ __forceinline__ int value_bin(float v, float max_s) {
    const float d = (max_s - v) * 8.f;
    return d < 255.f ? (int)d : 255;  // (also what is not a number or infinitely far)
}
__device__ __forceinline__ unsigned long long measure_of(float v, float max_s, bool by_mass) {
    return by_mass ? (unsigned long long)(expf(v - max_s) * kMassOneF) : 1ull;
}

// f(value) for every logit of the row, 16 bytes per load where the row allows it: a pass is bound by the latency of its
// loads (one block, 126 values per thread), so fewer and wider loads make it shorter.
template <typename F>
__device__ __forceinline__ void for_each_logit(const RowArgs& r, F f) {
    const int tid = threadIdx.x;
    int done = 0;
    if ((reinterpret_cast<uintptr_t>(r.z) & 15u) == 0) {
        const int n4 = r.vocab >> 2;
        const float4* z4 = reinterpret_cast<const float4*>(r.z);
#pragma unroll 2
        for (int i = tid; i < n4; i += kThreads) {
            const float4 x = __ldg(z4 + i);
            f(x.x), f(x.y), f(x.z), f(x.w);
        }
        done = n4 << 2;
    }
    for (int i = done + tid; i < r.vocab; i += kThreads) f(r.z[i]);
}

// One byte of the descent over the counts in tot[]: the lowest byte d with run + (bins above d) <= target.
__device__ __forceinline__ int lowest_byte(const unsigned long long* tot, unsigned long long target, unsigned long long* run) {
    int d = kBins - 1;
    while (d > 0 && *run + tot[d] <= target) { *run += tot[d]; --d; }
    return d;
}

__device__ unsigned radix_threshold(const RowArgs& r, float temp, float max_s, bool by_mass, double fraction,
                                    unsigned long long count_target, unsigned long long* hist, unsigned long long* tot,
                                    unsigned long long* sh, unsigned long long* above) {
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    // ---- pass 1: bins by value ----
    for (int i = tid; i < (kThreads / 32) * kBins; i += kThreads) hist[i] = 0ull;
    __syncthreads();
    unsigned long long* mine = hist + warp * kBins;
    unsigned long long far = 0ull;
    for_each_logit(r, [&](float zi) {
        const float v = zi / temp;
        const int b = value_bin(v, max_s);
        const unsigned long long w = measure_of(v, max_s, by_mass);
        if (b == kBins - 1) far += w;
        else atomicAdd(mine + b, w);
    });
    for (int o = 16; o > 0; o >>= 1) far += __shfl_xor_sync(0xffffffffu, far, o);
    if (lane == 0) mine[kBins - 1] = far;
    __syncthreads();
    if (tid < kBins) {
        unsigned long long t = 0ull;
        for (int w = 0; w < kThreads / 32; ++w) t += hist[w * kBins + tid];
        tot[tid] = t;
    }
    __syncthreads();
    if (tid == 0) {
        unsigned long long total = 0ull;
        for (int b = 0; b < kBins; ++b) total += tot[b];
        const unsigned long long target = by_mass ? (unsigned long long)((double)total * fraction) : count_target;
        // bins run from the highest values down: the threshold lies in the last bin d whose higher bins fit the target
        unsigned long long run = 0ull;
        int d = 0;
        while (d < kBins - 1 && run + tot[d] <= target) { run += tot[d]; ++d; }
        sh[0] = run, sh[1] = (unsigned long long)d, sh[2] = target;
        sh[3] = (d == kBins - 1 && run + tot[d] <= target) ? 1ull : 0ull;  // everything fits: every key is kept
        sh[4] = total;
    }
    __syncthreads();
    unsigned long long run_above = sh[0];
    const int bin = (int)sh[1];
    const unsigned long long target = sh[2];
    if (sh[3]) {
        *above = sh[4];
        __syncthreads();
        return 0u;
    }
    __syncthreads();
    // ---- pass 2: the keys of that bin, into the space of the warps' bins ----
    unsigned* list = reinterpret_cast<unsigned*>(hist);
    unsigned* n_list = reinterpret_cast<unsigned*>(sh + 5);
    bool listed = bin < kBins - 1;
    if (listed) {
        if (tid == 0) *n_list = 0u;
        __syncthreads();
        for_each_logit(r, [&](float zi) {
            const float v = zi / temp;
            if (value_bin(v, max_s) == bin) {
                const unsigned at = atomicAdd(n_list, 1u);
                if (at < (unsigned)kListCap) list[at] = order_key(v);
            }
        });
        __syncthreads();
        listed = *n_list <= (unsigned)kListCap;
    }
    const int n = listed ? (int)*n_list : 0;
    // ---- the threshold's four bytes: over the list, or over the row's values of that bin ----
    unsigned prefix = 0u;
    for (int level = 0; level < 4; ++level) {
        const int shift = 24 - 8 * level;
        if (tid < kBins) tot[tid] = 0ull;
        __syncthreads();
        if (listed) {
            for (int i = tid; i < n; i += kThreads) {
                const unsigned key = list[i];
                if (level == 0 || (key >> (shift + 8)) == (prefix >> (shift + 8)))
                    atomicAdd(tot + ((key >> shift) & 255u), measure_of(key_value(key), max_s, by_mass));
            }
        } else {
            for_each_logit(r, [&](float zi) {
                const float v = zi / temp;
                const unsigned key = order_key(v);
                if (value_bin(v, max_s) == bin && (level == 0 || (key >> (shift + 8)) == (prefix >> (shift + 8))))
                    atomicAdd(tot + ((key >> shift) & 255u), measure_of(v, max_s, by_mass));
            });
        }
        __syncthreads();
        if (tid == 0) {
            unsigned long long run = run_above;
            sh[1] = (unsigned long long)lowest_byte(tot, target, &run);
            sh[0] = run;
        }
        __syncthreads();
        run_above = sh[0];
        prefix |= (unsigned)sh[1] << shift;
        __syncthreads();
    }
    *above = run_above;
    return prefix;
}

constexpr int kChunks = 16;        // blocks that share one row in the first pass
constexpr int kPartialThreads = 256;

// First pass, (row, chunk) per block: maximum, its lowest index, and the sum of exp(z - maximum)
// over one sixteenth of the vocabulary.  The row kernel merges the sixteen results, so a greedy row
// needs no pass of its own over the logits.  partial[row][chunk] = {max, sum, index as float bits}.
__global__ void __launch_bounds__(kPartialThreads)
sample_partial_kernel(const float* __restrict__ logits, long long ld, int vocab, float* __restrict__ partial) {
    ns_pdl_launch_dependents();
    ns_pdl_wait();
    __shared__ float fscratch[32];
    __shared__ float smax[32];
    __shared__ int sidx[32];
    const int row = blockIdx.x, chunk = blockIdx.y;
    const float* z = logits + (size_t)row * ld;
    const int per = (vocab + kChunks - 1) / kChunks;
    const int lo = min(chunk * per, vocab), hi = min(lo + per, vocab);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    float best = -INFINITY;
    int besti = 0x7fffffff;
    for (int i = lo + tid; i < hi; i += kPartialThreads) {
        const float v = z[i];
        if (v > best || (v == best && i < besti)) { best = v; besti = i; }
    }
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, besti, o);
        if (ov > best || (ov == best && oi < besti)) { best = ov; besti = oi; }
    }
    if (lane == 0) { smax[warp] = best; sidx[warp] = besti; }
    __syncthreads();
    if (warp == 0) {
        best = lane < kPartialThreads / 32 ? smax[lane] : -INFINITY;
        besti = lane < kPartialThreads / 32 ? sidx[lane] : 0x7fffffff;
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, besti, o);
            if (ov > best || (ov == best && oi < besti)) { best = ov; besti = oi; }
        }
        if (lane == 0) { smax[0] = best; sidx[0] = besti; }
    }
    __syncthreads();
    const float cmax = smax[0];
    float se = 0.f;
    for (int i = lo + tid; i < hi; i += kPartialThreads) se += expf(z[i] - cmax);
    const float total = ns_block_sum(se, fscratch);
    if (tid == 0) {
        float* p = partial + ((size_t)row * kChunks + chunk) * 3;
        p[0] = cmax;
        p[1] = lo < hi ? total : 0.f;
        p[2] = __int_as_float(sidx[0]);
    }
}

__global__ void __launch_bounds__(kThreads)
sample_rows_kernel(const float* __restrict__ logits, long long ld, int vocab, const float* __restrict__ temperature,
                   const int* __restrict__ top_k, const float* __restrict__ top_p, const float* __restrict__ u,
                   const float* __restrict__ partial, int* __restrict__ token, float* __restrict__ logprob_raw,
                   float* __restrict__ logprob_proc) {
    ns_pdl_launch_dependents();  // the next kernel may be scheduled now; it waits for this one before it reads
    ns_pdl_wait();               // everything below sees the previous kernel's results
    __shared__ float fscratch[32];
    __shared__ float seg_prefix[kThreads];
    __shared__ int seg_eq_prefix[kThreads];
    __shared__ int found, last_kept;
    __shared__ float smax[32];
    __shared__ int sidx[32];
    __shared__ unsigned long long bin_total[kBins];
    __shared__ unsigned long long descent[6];
    extern __shared__ unsigned long long warp_bins[];  // [warps][kBins]

    const int row = blockIdx.x;
    const float* z = logits + (size_t)row * ld;
    const RowArgs r{z, vocab};
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    (void)lane;

    // ---- raw max, argmax (lowest index on ties) and log-sum-exp: merged from the first pass ------
    if (tid == 0) {
        const float* p = partial + (size_t)row * kChunks * 3;
        float best = -INFINITY;
        int besti = 0x7fffffff;
        for (int c = 0; c < kChunks; ++c) {  // chunks are in index order: the first maximum wins a tie
            const float v = p[3 * c];
            if (v > best) { best = v; besti = __float_as_int(p[3 * c + 2]); }
        }
        float se = 0.f;
        for (int c = 0; c < kChunks; ++c)
            if (p[3 * c + 1] > 0.f) se += p[3 * c + 1] * expf(p[3 * c] - best);
        smax[0] = best;
        sidx[0] = besti;
        fscratch[1] = logf(se) + best;
    }
    __syncthreads();
    const float zmax = smax[0];
    const int amax = sidx[0];
    const float lse_raw = fscratch[1];
    __syncthreads();  // fscratch is reused by the block sums below

    const float temp = temperature[row];
    if (!(temp > 0.f)) {  // greedy
        if (tid == 0) {
            token[row] = amax;
            logprob_raw[row] = zmax - lse_raw;
            logprob_proc[row] = 0.f;
        }
        return;
    }

    // ---- processed distribution ---------------------------------------------------------
    const float max_s = zmax / temp;
    const int k = top_k[row];
    const float p_keep = top_p[row];
    const bool nucleus = (k > 0 && k < vocab) || p_keep < 1.f;

    // Kept set: key > tau, plus the first n_eq tokens (by index) with key == tau.
    unsigned tau = 0u;       // every finite logit has key > 0
    int n_eq = 0x7fffffff;   // all tokens equal to tau
    if (nucleus) {
        unsigned tau_p = 0u;
        if (p_keep < 1.f) {
            // smallest key t with mass(key > t) <= top_p of the row's softmax mass (the reference sorts, takes the softmax of
            // all and keeps a token while the mass before it is <= top_p, spec/sampling.py:29-33); kept by top-p =
            // {key >= t}.  Logits that tie exactly at t are all kept: the reference's descending sort keeps whichever of them
            // it happens to place first, which no order of the vocabulary decides
            unsigned long long above;
            tau_p = radix_threshold(r, temp, max_s, true, (double)fmaxf(p_keep, 0.f), 0ull, warp_bins, bin_total, descent, &above);
        }
        unsigned tau_k = 0u;
        int eq_k = 0x7fffffff;
        if (k > 0 && k < vocab) {
            // k-th largest key: smallest t with count(key > t) <= k - 1; the tokens equal to it fill the k places that are left
            unsigned long long above;
            tau_k = radix_threshold(r, temp, max_s, false, 0.0, (unsigned long long)(k - 1), warp_bins, bin_total, descent, &above);
            eq_k = k - (int)above;
        }
        // combine: both kept sets are prefixes of the descending order; take the shorter one
        if (k > 0 && k < vocab && tau_k >= tau_p) {
            tau = tau_k;
            n_eq = eq_k;
        } else {
            // top-p alone decides: keep every key >= tau_p
            tau = tau_p > 0u ? tau_p - 1u : 0u;
            n_eq = 0;  // nothing equals tau_p - 1 that should be kept specially; keys > tau cover key >= tau_p
            if (tau_p == 0u) n_eq = 0x7fffffff;
        }
    }

    // ---- contiguous segments per thread: rank of tokens equal to tau, kept mass, draw -----
    const int seg = (vocab + kThreads - 1) / kThreads;
    const int s0 = min(tid * seg, vocab), s1 = min(s0 + seg, vocab);

    // index rank among tokens whose key == tau (needed only when n_eq is a real limit)
    int eq_before = 0;
    const bool limit_eq = nucleus && n_eq != 0x7fffffff && n_eq > 0;
    if (limit_eq) {
        int c = 0;
        for (int i = s0; i < s1; ++i)
            if (order_key(z[i] / temp) == tau) ++c;
        seg_eq_prefix[tid] = c;
        __syncthreads();
        if (tid == 0) {
            int run = 0;
            for (int t = 0; t < kThreads; ++t) { const int v = seg_eq_prefix[t]; seg_eq_prefix[t] = run; run += v; }
        }
        __syncthreads();
        eq_before = seg_eq_prefix[tid];
    }

    auto kept = [&](int i, float v, int& eq_seen) -> bool {
        if (!nucleus) return true;
        const unsigned key = order_key(v);
        if (key > tau) return true;
        if (key == tau && n_eq > 0) {
            if (n_eq == 0x7fffffff) return true;
            const bool ok = (eq_before + eq_seen) < n_eq;
            ++eq_seen;
            return ok;
        }
        return false;
    };

    // One pass for the kept tokens' weights exp(v - max_s): their sum per segment (exclusive prefix in thread order below)
    // and each thread's last kept token.  The draw compares running sums of the same weights with u x their total, so
    // the normalised probabilities are never formed.
    float segsum = 0.f;
    int last = -1;
    {
        int eq_seen = 0;
        for (int i = s0; i < s1; ++i) {
            const float v = z[i] / temp;
            if (kept(i, v, eq_seen)) {
                segsum += expf(v - max_s);
                last = i;
            }
        }
    }
    seg_prefix[tid] = segsum;
    if (tid == 0) { found = 0x7fffffff; last_kept = 0; }
    __syncthreads();
    if (last >= 0) atomicMax(&last_kept, last);  // used only if no thread's sum passes the target
    if (warp == 0) {
        // 32 consecutive segments per lane, then a warp scan of the lane totals
        float local = 0.f;
        for (int t = 0; t < 32; ++t) local += seg_prefix[lane * 32 + t];
        float incl = local;
        for (int o = 1; o < 32; o <<= 1) {
            const float up = __shfl_up_sync(0xffffffffu, incl, o);
            if (lane >= o) incl += up;
        }
        float run = incl - local;
        for (int t = 0; t < 32; ++t) {
            const float v = seg_prefix[lane * 32 + t];
            seg_prefix[lane * 32 + t] = run;
            run += v;
        }
        if (lane == 31) fscratch[0] = run;  // total
    }
    __syncthreads();
    const float total = fscratch[0];
    const float lse_s = logf(total) + max_s;
    const float target = u[row] * total;
    {
        // The running sum is compared with the target only right after a kept token has been added: a token outside
        // the set can never be reported, whatever the rounding of the scanned prefix.  A segment whose sum ends clearly
        // below the target cannot hold the crossing and is not walked again; one that starts above it reports its
        // first kept token at once (the smallest index reported wins).
        const float begin = seg_prefix[tid];
        if (segsum > 0.f && !(begin + segsum < target - 1e-4f * total)) {
            float run = begin;
            int eq_seen = 0;
            for (int i = s0; i < s1; ++i) {
                const float v = z[i] / temp;
                if (kept(i, v, eq_seen)) {
                    run += expf(v - max_s);
                    if (run > target) { atomicMin(&found, i); break; }
                }
            }
        }
    }
    __syncthreads();
    if (tid == 0) {
        int t = found;
        if (t > vocab - 1) t = last_kept;  // rounding left the target at or past the total: the last token of the set
        token[row] = t;
        logprob_raw[row] = z[t] - lse_raw;
        const float v = z[t] / temp;
        // (an empty set cannot occur: the largest logit is always kept)
        bool in_set = true;
        if (nucleus) {
            const unsigned key = order_key(v);
            in_set = key > tau || (key == tau && n_eq > 0);
        }
        logprob_proc[row] = in_set ? v - lse_s : -INFINITY;
    }
}

}  // namespace

// `partial`: scratch of n_rows * 16 * 3 floats for the first pass.
NS_API int ns_sample_rows(const float* logits, long long ld, int n_rows, int vocab, const float* temperature,
                          const int* top_k, const float* top_p, const float* u, float* partial, int* token,
                          float* logprob_raw, float* logprob_proc, cudaStream_t stream) {
    if (n_rows <= 0) return NS_OK;
    if (vocab <= 0) NS_FAIL(NS_ERR_ARGUMENT, "ns_sample_rows: vocab=%d", vocab);
    if (!partial) NS_FAIL(NS_ERR_ARGUMENT, "ns_sample_rows: no scratch for the first pass");
    NS_LAUNCH((sample_partial_kernel), dim3(n_rows, kChunks), kPartialThreads, 0, stream, logits, ld, vocab, partial);
    constexpr int kBinBytes = (kThreads / 32) * kBins * (int)sizeof(unsigned long long);
    static bool configured = false;
    if (!configured) {
        NS_CUDA(cudaFuncSetAttribute(sample_rows_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kBinBytes));
        configured = true;
    }
    NS_LAUNCH((sample_rows_kernel), n_rows, kThreads, kBinBytes, stream, logits, ld, vocab, temperature, top_k, top_p, u,
              (const float*)partial, token, logprob_raw, logprob_proc);
    NS_CHECK_LAUNCH("ns_sample_rows");
    return NS_OK;
}
