// Similarity-based row reordering (host engine, multi-threaded).
//
// Produces exactly what the reference program Matrix_Blocking writes when SMaT runs it as
// `-a 5 -b <col_block> -B <row_block> -F 1 -t <tau>` (src/reorder.py:131-132):
//   BlockingEngine::GetGrouping            preprocess/src/general/blocking.cpp:616-657
//     -> IterativeBlockingKeeper           preprocess/src/general/blocking.cpp:431-547
//          JaccardDistanceGroup            preprocess/src/general/blocking.cpp:904-975
//          merge_rows                      preprocess/src/general/utilities.cpp:145-173
//     -> get_fixed_size_grouping           preprocess/src/general/utilities.cpp:45-54
//   CSR::reorder -> get_permutation        preprocess/src/general/csr.cpp:97-105, utilities.cpp:8-20
//
// What is reproduced bit for bit, and how:
//   * the greedy scan order, the stale-distance pruning test and the `distances` array whose element
//     0 starts at -1 and all others at 0 (blocking.cpp:434, 467-471);
//   * merge_rows, which is not a set union: pattern entries beyond the position reached for the last
//     column of the merged row are dropped (utilities.cpp:145-173);
//   * the candidate set: a std::set<pair<float,long>> that the reference trims with
//     `it = end(); advance(it, k); erase(it, end())` (blocking.cpp:504-510).  Stepping past end() of
//     a libstdc++ red-black tree cycles header -> leftmost-of-rightmost -> ... -> header, so the call
//     erases the last 0, 1 or 2 elements depending on k and on whether the rightmost node has a left
//     child.  The same container type is used here, the landing position is computed from the node
//     links, and the same range-erase is issued, so the tree evolves identically;
//   * both argsorts use libstdc++'s unstable std::sort with the reference's comparator
//     (utilities.cpp:10-17), which fixes the order of rows inside a group.
//
// What is different: the Jaccard distance is evaluated on per-row lists of distinct column-block
// ids against a byte map of the pattern's column blocks (the value depends only on three counts,
// so it is the same float), and the distance evaluations of a scan are computed ahead in parallel
// windows by a thread pool; a merge invalidates the rest of the window, which is then recomputed.
// The reference passes the pattern vector by value to every distance call (blocking.cpp:904) and is
// single-threaded.
#include <stdint.h>
#include <string.h>

#include <algorithm>
#include <atomic>
#include <cmath>
#include <functional>
#include <numeric>
#include <set>
#include <thread>
#include <vector>

#include "smat_internal.h"

namespace smat {
namespace {

// Minimal fork-join pool: workers spin (with yields) on a generation counter.
class Pool {
   public:
    explicit Pool(int n) : n_(n < 1 ? 1 : n) {
        for (int t = 1; t < n_; t++) workers_.emplace_back([this, t] { loop(t); });
    }
    ~Pool() {
        stop_.store(true);
        gen_.fetch_add(1);
        for (auto& w : workers_) w.join();
    }
    int size() const { return n_; }
    // fn(tid) runs once on every thread (tid 0 = caller).
    void run(const std::function<void(int)>& fn) {
        if (n_ == 1) { fn(0); return; }
        fn_ = &fn;
        pending_.store(n_ - 1);
        gen_.fetch_add(1);
        fn(0);
        int spins = 0;
        while (pending_.load(std::memory_order_acquire) != 0)
            if (++spins > 64) std::this_thread::yield();
    }

   private:
    void loop(int tid) {
        uint64_t seen = 0;
        for (;;) {
            int spins = 0;
            uint64_t g;
            while ((g = gen_.load(std::memory_order_acquire)) == seen) {
                if (++spins > 256) { std::this_thread::yield(); }
            }
            seen = g;
            if (stop_.load()) return;
            (*fn_)(tid);
            pending_.fetch_sub(1, std::memory_order_release);
        }
    }
    int n_;
    std::vector<std::thread> workers_;
    std::atomic<uint64_t> gen_{0};
    std::atomic<int> pending_{0};
    std::atomic<bool> stop_{false};
    const std::function<void(int)>* fn_ = nullptr;
};

inline float jaccard_from_counts(int64_t sizeA, int64_t sizeB, int64_t nA, int64_t nB, int64_t nAB, int64_t gA) {
    // JaccardDistanceGroup with group_size_B = 1 and count_zeros = 1 (blocking.cpp:904-975)
    if (sizeA == 0 && sizeB == 0) return 0.0f;
    if (sizeA == 0 || sizeB == 0) return 1.0f;
    const int64_t count = (nA - nAB) * 1 + (nB - nAB) * gA;
    return (float)((2.0 * (double)count) / (double)(nA * gA + nB * 1 + count));
}

struct Engine {
    int64_t rows;
    const int64_t* rowptr;
    const int32_t* cols;
    int64_t cb;
    // distinct column-block ids per row
    std::vector<int64_t> bptr;
    std::vector<int32_t> bids;
    int64_t n_colblocks = 0;

    void build_block_lists(Pool& pool) {
        bptr.assign((size_t)rows + 1, 0);
        // pass 1: counts
        pool.run([&](int tid) {
            const int64_t lo = rows * tid / pool.size(), hi = rows * (tid + 1) / pool.size();
            for (int64_t r = lo; r < hi; r++) {
                int64_t n = 0, last = -1;
                for (int64_t j = rowptr[r]; j < rowptr[r + 1]; j++) {
                    const int64_t b = cols[j] / cb;
                    if (b != last) { n++; last = b; }
                }
                bptr[(size_t)r + 1] = n;
            }
        });
        for (int64_t r = 0; r < rows; r++) bptr[(size_t)r + 1] += bptr[(size_t)r];
        bids.resize((size_t)bptr[(size_t)rows]);
        std::vector<int64_t> maxb((size_t)pool.size(), -1);
        pool.run([&](int tid) {
            const int64_t lo = rows * tid / pool.size(), hi = rows * (tid + 1) / pool.size();
            int64_t mb = -1;
            for (int64_t r = lo; r < hi; r++) {
                int64_t at = bptr[(size_t)r], last = -1;
                for (int64_t j = rowptr[r]; j < rowptr[r + 1]; j++) {
                    const int64_t b = cols[j] / cb;
                    if (b != last) { bids[(size_t)at++] = (int32_t)b; last = b; if (b > mb) mb = b; }
                }
            }
            maxb[(size_t)tid] = mb;
        });
        n_colblocks = *std::max_element(maxb.begin(), maxb.end()) + 1;
    }
};

}  // namespace
}  // namespace smat

using namespace smat;


#ifndef __GLIBCXX__
#error "reorder.cpp reproduces a libstdc++-specific effect of the reference (see trim_count); build it with libstdc++"
#endif

namespace {
using CandSet = std::set<std::pair<float, long>>;

// The reference trims its candidate set with `it = end(); advance(it, k); erase(it, end())`
// (preprocess/src/general/blocking.cpp:504-510): it steps PAST end().  With libstdc++'s red-black tree, incrementing
// from the header node goes to the rightmost node's subtree and cycles through the header, the rightmost node and (when
// it has one) its left child, so the walk lands 0, 1 or 2 nodes before end() depending on k and on whether the rightmost
// node has a left child.  This returns how many of the largest candidates that erase removes; it reads the tree's
// node links, which is what the self-test below guards.
inline int64_t trim_count(const CandSet& best, int64_t k) {
    auto hdr = best.end()._M_node;
    const bool has_left = hdr->_M_right->_M_left != nullptr;
    const int64_t cyc = has_left ? 3 : 2;
    const int64_t pos = k % cyc;
    return pos ? cyc - pos : 0;
}

// First-call check that the model above is what this standard library does: for small sets, really walk k steps past
// end() the way the reference does and compare the distance to end() with trim_count.  A library with another tree
// layout fails here, loudly, instead of producing a different grouping.
bool trim_model_holds() {
    for (int n = 1; n <= 9; n++) {
        CandSet s;
        for (int i = 0; i < n; i++) s.insert({(float)((i * 7) % 11), (long)i});
        for (int64_t k = 0; k <= 7; k++) {
            auto it = s.end();
            for (int64_t i = 0; i < k; i++) ++it;  // the reference's std::advance(it, k) from end()
            int64_t dist = 0;
            for (auto e = it; e != s.end() && dist <= n; ++e) dist++;
            if (dist != trim_count(s, k)) return false;
        }
    }
    return true;
}
}  // namespace

extern "C" {

float smat_jaccard_group(const int64_t* rowA, size_t sizeA, int64_t gA, const int64_t* rowB, size_t sizeB, int64_t gB,
                         int64_t bs) {
    if (sizeA == 0 && sizeB == 0) return 0.0f;
    if (sizeA == 0 || sizeB == 0) return 1.0f;
    // distinct block counts of both lists and of their intersection (both lists ascending)
    size_t i = 0, j = 0;
    int64_t nA = 0, nB = 0, nAB = 0;
    while (i < sizeA || j < sizeB) {
        const int64_t pa = i < sizeA ? rowA[i] / bs : INT64_MAX;
        const int64_t pb = j < sizeB ? rowB[j] / bs : INT64_MAX;
        const int64_t p = pa < pb ? pa : pb;
        if (pa == p) { nA++; while (i < sizeA && rowA[i] / bs == p) i++; }
        if (pb == p) { nB++; while (j < sizeB && rowB[j] / bs == p) j++; }
        if (pa == p && pb == p) nAB++;
    }
    const int64_t count = (nA - nAB) * gB + (nB - nAB) * gA;
    return (float)((2.0 * (double)count) / (double)(nA * gA + nB * gB + count));
}

}  // extern "C"

namespace {

// The clustering, then either the fixed-size regrouping of the reference's -F 1 (fixed) or the grouping as the
// clustering leaves it (numbers of full groups lowered by the row count, as the reference does), and the
// permutation get_permutation derives from whichever it is.
int reorder_impl(size_t rows_, const int64_t* rowptr, const int32_t* cols, float tau, int col_block, int row_block, int threads,
                 bool fixed_size, int64_t* grouping_out, int64_t* perm_out) {
    clear_error();
    if ((rows_ && (!rowptr || !grouping_out)) || col_block < 1 || row_block < 1)
        return fail(SMAT_ERR_BAD_ARG, "bad argument");
    const int64_t rows = (int64_t)rows_;
    if (rows == 0) return SMAT_OK;
    static const bool model_ok = trim_model_holds();
    if (!model_ok)
        return fail(SMAT_ERR_RANGE, "this C++ standard library's std::set does not behave like the one the reference's "
                                    "candidate trim was characterised with; groupings would differ from the reference");
    if (rowptr[rows] > 0 && !cols) return fail(SMAT_ERR_BAD_ARG, "cols is NULL");
    for (int64_t r = 0; r < rows; r++)
        for (int64_t j = rowptr[r] + 1; j < rowptr[r + 1]; j++)
            if (cols[j] < cols[j - 1]) return fail(SMAT_ERR_BAD_ARG, "row %lld: columns must be ascending", (long long)r);
    if (threads <= 0) threads = (int)std::thread::hardware_concurrency();
    if (threads < 1) threads = 1;
    if (threads > 64) threads = 64;
    Pool pool(threads);

    Engine E;
    E.rows = rows;
    E.rowptr = rowptr;
    E.cols = cols;
    E.cb = col_block;
    E.build_block_lists(pool);

    const int64_t maxg = row_block;
    std::vector<int64_t> grouping((size_t)rows, -1);
    std::vector<float> distances((size_t)rows, 0.0f);
    distances[0] = -1.0f;
    std::vector<uint8_t> inpat((size_t)E.n_colblocks + 1, 0);
    std::vector<float> wdist;   // distances computed ahead for the current window
    std::vector<int32_t> pattern, merged_tmp;
    std::vector<int64_t> merged;

    for (int64_t i = 0; i < rows; i++) {
        if (grouping[(size_t)i] != -1) continue;
        std::set<std::pair<float, long>> best;
        merged.clear();
        const int64_t group_number = i + rows;
        int64_t gsize = 1;
        grouping[(size_t)i] = group_number;
        merged.push_back(i);
        pattern.assign(cols + rowptr[i], cols + rowptr[i + 1]);
        // pattern block map
        int64_t nA = 0;
        auto rebuild_map = [&](bool set) {
            int64_t last = -1, n = 0;
            for (int32_t c : pattern) {
                const int64_t b = c / col_block;
                if (b != last) { inpat[(size_t)b] = set ? 1 : 0; n++; last = b; }
            }
            if (set) nA = n;
        };
        // the pattern can hold columns beyond the largest block id seen in any row? No: it only ever
        // holds columns of rows, so every block id is < n_colblocks.
        rebuild_map(true);
        const float di = distances[(size_t)i];

        int64_t j = i + 1;
        int64_t window = 256;
        while (j < rows && gsize != maxg) {
            const int64_t wstart = j;
            const int64_t wend = std::min(rows, j + window);
            const int64_t wn = wend - j;
            wdist.resize((size_t)wn);
            const int64_t sizeA = (int64_t)pattern.size();
            const int64_t gA = gsize;
            auto eval = [&](int64_t lo, int64_t hi) {
                for (int64_t x = lo; x < hi; x++) {
                    const int64_t jj = wstart + x;
                    const float dj = distances[(size_t)jj];
                    if ((di != -1 && dj != -1 && std::abs(di - dj) > tau) || grouping[(size_t)jj] != -1) continue;
                    int64_t nAB = 0;
                    const int64_t b0 = E.bptr[(size_t)jj], b1 = E.bptr[(size_t)jj + 1];
                    for (int64_t k = b0; k < b1; k++) nAB += inpat[(size_t)E.bids[(size_t)k]];
                    wdist[(size_t)x] = jaccard_from_counts(sizeA, rowptr[jj + 1] - rowptr[jj], nA, b1 - b0, nAB, gA);
                }
            };
            if (wn >= 2048 && pool.size() > 1) {
                pool.run([&](int tid) { eval(wn * tid / pool.size(), wn * (tid + 1) / pool.size()); });
            } else {
                eval(0, wn);
            }
            bool merged_here = false;
            for (; j < wend; j++) {
                if (gsize == maxg) break;
                const float dj = distances[(size_t)j];
                if (di != -1 && dj != -1 && std::abs(di - dj) > tau) {
                    distances[(size_t)j] = -1;
                    continue;
                }
                if (grouping[(size_t)j] != -1) continue;
                const float dist = wdist[(size_t)(j - wstart)];
                distances[(size_t)j] = dist;
                if (dist <= tau) {
                    grouping[(size_t)j] = group_number;
                    merged.push_back(j);
                    // merge_rows as the reference performs it (tail of the pattern may be dropped)
                    rebuild_map(false);
                    merged_tmp.clear();
                    {
                        const int32_t* Bp = cols + rowptr[j];
                        const int64_t sizeB = rowptr[j + 1] - rowptr[j];
                        size_t ia = 0;
                        int64_t jb = 0;
                        while (jb < sizeB) {
                            const int32_t bval = Bp[jb];
                            const size_t ni =
                                (size_t)(std::lower_bound(pattern.begin() + (long)ia, pattern.end(), bval) - pattern.begin());
                            if (ni == pattern.size()) break;
                            merged_tmp.insert(merged_tmp.end(), pattern.begin() + (long)ia, pattern.begin() + (long)ni);
                            merged_tmp.push_back(bval);
                            ia = (pattern[ni] == bval) ? ni + 1 : ni;
                            jb++;
                        }
                        merged_tmp.insert(merged_tmp.end(), Bp + jb, Bp + sizeB);
                    }
                    pattern.swap(merged_tmp);
                    rebuild_map(true);
                    gsize++;
                    j++;
                    merged_here = true;
                    break;  // the rest of the window was computed against the old pattern
                } else {
                    best.insert({dist, (long)j});
                    const int64_t k = maxg - (int64_t)merged.size();
                    if ((int64_t)best.size() > k) {
                        const int64_t n_erase = trim_count(best, k);
                        if (n_erase > 0) best.erase(std::prev(best.end(), n_erase), best.end());
                    }
                }
            }
            window = merged_here ? 256 : std::min<int64_t>(window * 4, 1 << 20);
        }
        rebuild_map(false);

        if (gsize < maxg) {
            for (auto it = best.begin(); it != best.end() && gsize != maxg; ++it) {
                grouping[(size_t)it->second] = group_number;
                merged.push_back(it->second);
                gsize++;
            }
        }
        if (gsize == maxg)
            for (int64_t idx : merged) grouping[(size_t)idx] -= rows;
    }

    // -F 1: fixed-size grouping, then the permutation CSR::reorder applies
    auto argsort = [&](const std::vector<int64_t>& key) {
        std::vector<int64_t> v((size_t)rows);
        std::iota(v.begin(), v.end(), 0);
        auto comp = [&](int a, int b) { return key[(size_t)a] < key[(size_t)b]; };
        std::sort(v.begin(), v.end(), comp);
        return v;
    };
    const std::vector<int64_t> p1 = argsort(grouping);
    if (!fixed_size) {
        memcpy(grouping_out, grouping.data(), (size_t)rows * sizeof(int64_t));
        if (perm_out) memcpy(perm_out, p1.data(), (size_t)rows * sizeof(int64_t));
        return SMAT_OK;
    }
    std::vector<int64_t> fixed((size_t)rows, -1);
    for (int64_t x = 0; x < rows; x++) fixed[(size_t)p1[(size_t)x]] = x / row_block;
    const std::vector<int64_t> p2 = argsort(fixed);
    memcpy(grouping_out, fixed.data(), (size_t)rows * sizeof(int64_t));
    if (perm_out) memcpy(perm_out, p2.data(), (size_t)rows * sizeof(int64_t));
    return SMAT_OK;
}

}  // namespace

extern "C" {

int smat_reorder_rows(size_t rows, const int64_t* rowptr, const int32_t* cols, float tau, int col_block, int row_block,
                      int threads, int64_t* grouping_out, int64_t* perm_out) {
    if (rows && !perm_out) {
        clear_error();
        return fail(SMAT_ERR_BAD_ARG, "bad argument");
    }
    return reorder_impl(rows, rowptr, cols, tau, col_block, row_block, threads, true, grouping_out, perm_out);
}

int smat_cluster_rows(size_t rows, const int64_t* rowptr, const int32_t* cols, float tau, int col_block, int max_group_rows,
                      int threads, int64_t* grouping_out, int64_t* perm_out) {
    return reorder_impl(rows, rowptr, cols, tau, col_block, max_group_rows, threads, false, grouping_out, perm_out);
}

}  // extern "C"
