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
// at the top-k boundary equal logits are taken in order of their index.
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

// sum over the row of exp(z / temp - max_s) for the tokens whose ordering key exceeds tau
__device__ float block_sum_if_key_gt(const RowArgs& r, float temp, float max_s, unsigned tau, float* scratch) {
    float s = 0.f;
    for (int i = threadIdx.x; i < r.vocab; i += kThreads) {
        const float v = r.z[i] / temp;
        if (order_key(v) > tau) s += expf(v - max_s);
    }
    return ns_block_sum(s, scratch);
}

__device__ int block_count_key_gt(const RowArgs& r, float temp, unsigned tau, int* iscratch) {
    int c = 0;
    for (int i = threadIdx.x; i < r.vocab; i += kThreads)
        if (order_key(r.z[i] / temp) > tau) ++c;
    // integer block sum
    for (int o = 16; o > 0; o >>= 1) c += __shfl_xor_sync(0xffffffffu, c, o);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) iscratch[threadIdx.x >> 5] = c;
    __syncthreads();
    int t = (threadIdx.x < kThreads / 32) ? iscratch[threadIdx.x] : 0;
    if (threadIdx.x < 32) {
        for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
        if (threadIdx.x == 0) iscratch[0] = t;
    }
    __syncthreads();
    return iscratch[0];
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
    __shared__ int iscratch[32];
    __shared__ float seg_prefix[kThreads];
    __shared__ int seg_eq_prefix[kThreads];
    __shared__ int found, last_kept;
    __shared__ float smax[32];
    __shared__ int sidx[32];

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
        // softmax denominator over the whole row (the reference sorts, then takes softmax of all)
        float s = 0.f;
        for (int i = tid; i < vocab; i += kThreads) s += expf(z[i] / temp - max_s);
        const float denom = ns_block_sum(s, fscratch);

        unsigned tau_p = 0u;
        if (p_keep < 1.f) {
            // smallest key t with mass(key > t) <= top_p; kept by top-p = {key >= t}.  Logits that tie exactly at t are
            // all kept: the reference's descending sort (spec/sampling.py:29-33) keeps whichever of them it happens to
            // place first, which no order of the vocabulary decides
            unsigned lo = 0u;  // bitwise descent: build the smallest t for which the predicate holds
            for (int bit = 31; bit >= 0; --bit) {
                // candidate with this bit cleared and all lower bits set is the largest value in the lower half
                const unsigned cand = lo | ((1u << bit) - 1u);
                const float mass = block_sum_if_key_gt(r, temp, max_s, cand, fscratch) / denom;
                if (!(mass <= p_keep)) lo |= (1u << bit);  // predicate false on the lower half's top: answer is above
            }
            tau_p = lo;  // kept = {key >= tau_p} = {key > tau_p - 1}
        }
        unsigned tau_k = 0u;
        int eq_k = 0x7fffffff;
        if (k > 0 && k < vocab) {
            // k-th largest key: smallest t with count(key > t) <= k - 1
            unsigned lo = 0u;
            for (int bit = 31; bit >= 0; --bit) {
                const unsigned cand = lo | ((1u << bit) - 1u);
                const int cnt = block_count_key_gt(r, temp, cand, iscratch);
                if (!(cnt <= k - 1)) lo |= (1u << bit);
            }
            tau_k = lo;
            eq_k = k - block_count_key_gt(r, temp, tau_k, iscratch);
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

    // kept log-sum-exp
    float ks = 0.f;
    {
        int eq_seen = 0;
        for (int i = s0; i < s1; ++i) {
            const float v = z[i] / temp;
            if (kept(i, v, eq_seen)) ks += expf(v - max_s);
        }
    }
    const float lse_s = logf(ns_block_sum(ks, fscratch)) + max_s;

    // segment sums of probabilities, exclusive prefix in thread order
    float segsum = 0.f;
    {
        int eq_seen = 0;
        for (int i = s0; i < s1; ++i) {
            const float v = z[i] / temp;
            if (kept(i, v, eq_seen)) segsum += expf(v - lse_s);
        }
    }
    seg_prefix[tid] = segsum;
    if (tid == 0) { found = 0x7fffffff; last_kept = 0; }
    __syncthreads();
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
    const float target = u[row] * total;
    {
        // the running sum is compared with the target only right after a kept token has been added: a token
        // outside the set can never be reported, whatever the rounding of the scanned prefix
        float run = seg_prefix[tid];
        int eq_seen = 0, last = -1;
        for (int i = s0; i < s1; ++i) {
            const float v = z[i] / temp;
            if (kept(i, v, eq_seen)) {
                run += expf(v - lse_s);
                last = i;
                if (run > target) { atomicMin(&found, i); break; }
            }
        }
        if (last >= 0) atomicMax(&last_kept, last);  // used only if no thread's sum passed the target
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
    NS_LAUNCH((sample_rows_kernel), n_rows, kThreads, 0, stream, logits, ld, vocab, temperature, top_k, top_p, u,
              (const float*)partial, token, logprob_raw, logprob_proc);
    NS_CHECK_LAUNCH("ns_sample_rows");
    return NS_OK;
}
