// Block manager for the paged KV pool, with a device-resident copy of the block tables.
//
// Host logic restated from runtime/src/cache/block.rs:84-346 of the reference (itself a port
// of the Python engine's block manager): a fixed pool of reference-counted physical blocks, a
// LIFO free list (`free_blocks.pop()`, :165 - the highest free id is handed out first, freed
// ids are reused most-recent-first), per-request ordered tables, prefix hits PREPENDED to a
// table (`assign_cached_blocks`, :214-232), `share_prefix` (:273-306), `ensure_blocks`
// (:236-268), single-block release for radix eviction (`free_block`, :200-210).
//
// What is new is the device mirror.  The reference rebuilds tables on the host every step;
// at 2048 requests x 2048 blocks that is a 16 MB upload per decode step.  Here every request
// owns a stable row of a caller-provided device array `[rows, max_blocks]` int32; `sync`
// uploads only the entries that changed since the last sync (normally one new block id per
// request every 16 steps), and the decode entry points read row `table_rows[r]` for batch
// position r, so batch order can change freely without touching the tables.

#include <algorithm>
#include <string>
#include <unordered_map>
#include <vector>

#include "sfb_common.cuh"

namespace {

struct Request {
    std::vector<int32_t> table;
    int64_t row = -1;         // row of the device mirror
    int64_t dirty_lo = 0;     // entries [dirty_lo, table.size()) differ from the device copy
};

}  // namespace

struct SFBBlockManager {
    int64_t num_blocks = 0, block_size = 0;
    std::vector<int32_t> ref_count;
    std::vector<int32_t> free_blocks;  // LIFO: back() is handed out next
    std::unordered_map<std::string, Request> requests;
    // device mirror
    int32_t* d_tables = nullptr;
    int64_t rows = 0, max_blocks = 0;
    std::vector<int64_t> free_rows;
    // Changed entries travel as (flat index, block id) pairs in pinned host memory that the
    // scatter kernel reads in place; two buffers alternate so that filling one never waits
    // for the kernel that is still reading the other.
    struct Staging {
        int2* host = nullptr;
        int64_t capacity = 0;
        cudaEvent_t done = nullptr;
    } staging[2];
    int next_staging = 0;
    ~SFBBlockManager() {
        for (auto& st : staging) {
            if (st.done) { cudaEventSynchronize(st.done); cudaEventDestroy(st.done); }
            if (st.host) cudaFreeHost(st.host);
        }
    }
};

using namespace sfb;

namespace {

__global__ void table_scatter_kernel(const int2* __restrict__ pairs, int64_t n, int32_t* __restrict__ tables) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) {
        const int2 p = pairs[i];
        tables[p.x] = p.y;
    }
}

int oom(const SFBBlockManager* bm, int64_t needed) {
    return fail(SFB_ERR_OUT_OF_BLOCKS, "OutOfMemory: need %lld blocks but only %lld free (total pool: %lld)", (long long)needed,
                (long long)bm->free_blocks.size(), (long long)bm->num_blocks);
}

int take_row(SFBBlockManager* bm, Request& r) {
    if (!bm->d_tables || r.row >= 0) return SFB_OK;
    if (bm->free_rows.empty()) return fail(SFB_ERR_OUT_OF_BLOCKS, "block manager: all %lld device table rows are in use", (long long)bm->rows);
    r.row = bm->free_rows.back();
    bm->free_rows.pop_back();
    r.dirty_lo = 0;
    return SFB_OK;
}

int32_t pop_block(SFBBlockManager* bm) {
    const int32_t bid = bm->free_blocks.back();
    bm->free_blocks.pop_back();
    bm->ref_count[bid] += 1;
    return bid;
}

}  // namespace

extern "C" {

SFBBlockManager* sfb_bm_create(int64_t num_blocks, int64_t block_size) {
    if (num_blocks <= 0 || block_size <= 0 || num_blocks > 0x7fffffffLL) {  // block.rs:93-99
        set_error("block manager: num_blocks and block_size must be positive");
        return nullptr;
    }
    auto* bm = new SFBBlockManager();
    bm->num_blocks = num_blocks;
    bm->block_size = block_size;
    bm->ref_count.assign((size_t)num_blocks, 0);
    bm->free_blocks.resize((size_t)num_blocks);
    for (int64_t i = 0; i < num_blocks; ++i) bm->free_blocks[(size_t)i] = (int32_t)i;  // (0..num_blocks).collect(), :107
    return bm;
}

void sfb_bm_destroy(SFBBlockManager* bm) { delete bm; }

int sfb_bm_attach_device_tables(SFBBlockManager* bm, void* d_tables, int64_t rows, int64_t max_blocks) {
    if (!bm || !d_tables || rows <= 0 || max_blocks <= 0 || rows > 0x7fffffffLL / max_blocks)
        return fail(SFB_ERR_INVALID_ARG, "block manager: bad device table arguments");
    if (!bm->requests.empty()) return fail(SFB_ERR_INVALID_ARG, "block manager: attach the device tables before the first allocation");
    bm->d_tables = static_cast<int32_t*>(d_tables);
    bm->rows = rows;
    bm->max_blocks = max_blocks;
    bm->free_rows.clear();
    for (int64_t r = rows - 1; r >= 0; --r) bm->free_rows.push_back(r);
    return SFB_OK;
}

// block.rs:146-172.  Writes the allocated ids to `out` (capacity `cap`); returns their count or a negative status.
int64_t sfb_bm_allocate(SFBBlockManager* bm, const char* rid, int64_t num_tokens, int32_t* out, int64_t cap) {
    if (!bm || !rid || num_tokens < 0) return fail(SFB_ERR_INVALID_ARG, "block manager: bad allocate arguments");
    if (bm->requests.count(rid)) return oom(bm, 0);  // an existing request is refused the same way (:147-153)
    const int64_t needed = ceil_div(num_tokens, bm->block_size);
    if (needed > (int64_t)bm->free_blocks.size()) return oom(bm, needed);
    if (bm->d_tables && needed > bm->max_blocks) return fail(SFB_ERR_INVALID_ARG, "block manager: %lld blocks exceed the device table width %lld", (long long)needed, (long long)bm->max_blocks);
    Request r;
    int rc = take_row(bm, r);
    if (rc) return rc;
    for (int64_t i = 0; i < needed; ++i) r.table.push_back(pop_block(bm));
    if (out)
        for (int64_t i = 0; i < needed && i < cap; ++i) out[i] = r.table[(size_t)i];
    bm->requests.emplace(rid, std::move(r));
    return needed;
}

// block.rs:176-195
void sfb_bm_free(SFBBlockManager* bm, const char* rid) {
    if (!bm || !rid) return;
    auto it = bm->requests.find(rid);
    if (it == bm->requests.end()) return;
    for (int32_t bid : it->second.table) {
        if (bid < 0 || bid >= bm->num_blocks) continue;  // ids assign_cached_blocks took from outside the pool: skipped like :184
        int32_t& rc = bm->ref_count[(size_t)bid];
        rc = rc > 0 ? rc - 1 : 0;
        if (rc == 0) bm->free_blocks.push_back(bid);
    }
    if (it->second.row >= 0) bm->free_rows.push_back(it->second.row);
    bm->requests.erase(it);
}

// block.rs:198-210
void sfb_bm_free_block(SFBBlockManager* bm, int64_t block_id) {
    if (!bm || block_id < 0 || block_id >= bm->num_blocks) return;
    int32_t& rc = bm->ref_count[(size_t)block_id];
    rc = rc > 0 ? rc - 1 : 0;
    if (rc == 0) bm->free_blocks.push_back((int32_t)block_id);
}

// block.rs:214-232: reference counts go up, the ids are put IN FRONT of the table
int sfb_bm_assign_cached_blocks(SFBBlockManager* bm, const char* rid, const int32_t* block_ids, int64_t n) {
    if (!bm || !rid || n < 0 || (n > 0 && !block_ids)) return fail(SFB_ERR_INVALID_ARG, "block manager: bad assign_cached_blocks arguments");
    auto known = bm->requests.find(rid);
    const int64_t have = known == bm->requests.end() ? 0 : (int64_t)known->second.table.size();
    if (bm->d_tables && have + n > bm->max_blocks)
        return fail(SFB_ERR_INVALID_ARG, "block manager: table would exceed the device table width");
    if (bm->d_tables && known == bm->requests.end() && bm->free_rows.empty())
        return fail(SFB_ERR_OUT_OF_BLOCKS, "block manager: all %lld device table rows are in use", (long long)bm->rows);
    Request& r = bm->requests[rid];
    int rc = take_row(bm, r);
    if (rc) return rc;
    for (int64_t i = 0; i < n; ++i)
        if (block_ids[i] >= 0 && block_ids[i] < bm->num_blocks) bm->ref_count[(size_t)block_ids[i]] += 1;
    r.table.insert(r.table.begin(), block_ids, block_ids + n);
    r.dirty_lo = 0;  // every entry moved
    return SFB_OK;
}

// block.rs:236-268
int sfb_bm_ensure_blocks(SFBBlockManager* bm, const char* rid, int64_t target_tokens) {
    if (!bm || !rid || target_tokens < 0) return fail(SFB_ERR_INVALID_ARG, "block manager: bad ensure_blocks arguments");
    auto it = bm->requests.find(rid);
    const int64_t existing = it == bm->requests.end() ? 0 : (int64_t)it->second.table.size() * bm->block_size;
    if (existing >= target_tokens) return SFB_OK;
    const int64_t n_extra = ceil_div(target_tokens - existing, bm->block_size);
    if (n_extra > (int64_t)bm->free_blocks.size()) return oom(bm, n_extra);
    if (bm->d_tables && existing / bm->block_size + n_extra > bm->max_blocks)
        return fail(SFB_ERR_INVALID_ARG, "block manager: table would exceed the device table width");
    if (bm->d_tables && it == bm->requests.end() && bm->free_rows.empty())
        return fail(SFB_ERR_OUT_OF_BLOCKS, "block manager: all %lld device table rows are in use", (long long)bm->rows);
    Request& r = bm->requests[rid];
    int rc = take_row(bm, r);
    if (rc) return rc;
    r.dirty_lo = std::min<int64_t>(r.dirty_lo, (int64_t)r.table.size());
    for (int64_t i = 0; i < n_extra; ++i) r.table.push_back(pop_block(bm));
    return SFB_OK;
}

// block.rs:273-306.  Returns the number of shared blocks or a negative status.
int64_t sfb_bm_share_prefix(SFBBlockManager* bm, const char* src, const char* dst, int64_t prefix_len) {
    if (!bm || !src || !dst || prefix_len < 0) return fail(SFB_ERR_INVALID_ARG, "block manager: bad share_prefix arguments");
    auto it = bm->requests.find(src);
    if (it == bm->requests.end()) return fail(SFB_ERR_INVALID_ARG, "Source request '%s' not found", src);
    if (bm->requests.count(dst)) return fail(SFB_ERR_INVALID_ARG, "Destination request '%s' already has blocks", dst);
    const int64_t n = ceil_div(prefix_len, bm->block_size);
    if (n > (int64_t)it->second.table.size())
        return fail(SFB_ERR_INVALID_ARG, "Source has %lld blocks, cannot share %lld (prefix_len=%lld, block_size=%lld)",
                    (long long)it->second.table.size(), (long long)n, (long long)prefix_len, (long long)bm->block_size);
    Request r;
    int rc = take_row(bm, r);
    if (rc) return rc;
    r.table.assign(it->second.table.begin(), it->second.table.begin() + n);
    for (int32_t bid : r.table) {
        if (bid < 0 || bid >= bm->num_blocks) {  // :292-294: the counts raised so far stay raised, the destination gets no table
            if (r.row >= 0) bm->free_rows.push_back(r.row);
            return fail(SFB_ERR_INVALID_ARG, "block %d not found in share_prefix", (int)bid);
        }
        bm->ref_count[(size_t)bid] += 1;
    }
    bm->requests.emplace(dst, std::move(r));
    return n;
}

void sfb_bm_increment_ref_count(SFBBlockManager* bm, int64_t block_id) {  // block.rs:330-334
    if (bm && block_id >= 0 && block_id < bm->num_blocks) bm->ref_count[(size_t)block_id] += 1;
}

int64_t sfb_bm_ref_count(const SFBBlockManager* bm, int64_t block_id) {
    return (bm && block_id >= 0 && block_id < bm->num_blocks) ? bm->ref_count[(size_t)block_id] : -1;
}

int64_t sfb_bm_num_free_blocks(const SFBBlockManager* bm) { return bm ? (int64_t)bm->free_blocks.size() : 0; }

// Copies the request's table to `out`; returns its length, or SFB_ERR_INVALID_ARG for an unknown request (block.rs:310-315).
int64_t sfb_bm_get_blocks(const SFBBlockManager* bm, const char* rid, int32_t* out, int64_t cap) {
    if (!bm || !rid) return SFB_ERR_INVALID_ARG;
    auto it = bm->requests.find(rid);
    if (it == bm->requests.end()) return fail(SFB_ERR_INVALID_ARG, "Unknown request_id: %s", rid);
    const auto& t = it->second.table;
    if (out)
        for (size_t i = 0; i < t.size() && (int64_t)i < cap; ++i) out[i] = t[i];
    return (int64_t)t.size();
}

// Row of the device mirror that holds this request's table (-1: unknown request or no mirror attached).
int64_t sfb_bm_row(const SFBBlockManager* bm, const char* rid) {
    if (!bm || !rid) return -1;
    auto it = bm->requests.find(rid);
    return it == bm->requests.end() ? -1 : it->second.row;
}

// block.rs:236-268 for a whole batch: the same as n calls in order; stops at the first failure (its index is in the message).
int sfb_bm_ensure_blocks_batch(SFBBlockManager* bm, const char* const* rids, const int64_t* target_tokens, int64_t n) {
    if (!bm || n < 0 || (n > 0 && (!rids || !target_tokens))) return fail(SFB_ERR_INVALID_ARG, "block manager: bad ensure_blocks_batch arguments");
    for (int64_t i = 0; i < n; ++i) {
        const int rc = sfb_bm_ensure_blocks(bm, rids[i], target_tokens[i]);
        if (rc) return rc;
    }
    return SFB_OK;
}

// Sends every table entry that changed since the previous sync to the device tables, as ONE kernel launch on
// `stream` that scatters (index, id) pairs out of pinned host memory.  Asynchronous: it only ever waits for the
// launch issued two syncs earlier (the one that last read the staging buffer it is about to refill).
// Returns the number of int32 entries sent.
int64_t sfb_bm_sync(SFBBlockManager* bm, void* stream) {
    if (!bm || !bm->d_tables) return fail(SFB_ERR_INVALID_ARG, "block manager: no device tables attached");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    int64_t total = 0;
    for (auto& kv : bm->requests)
        if (kv.second.row >= 0) total += std::max<int64_t>(0, (int64_t)kv.second.table.size() - kv.second.dirty_lo);
    if (total == 0) return 0;
    auto& buf = bm->staging[bm->next_staging];
    bm->next_staging ^= 1;
    if (buf.done) SFB_CUDA_CHECK(cudaEventSynchronize(buf.done));
    else SFB_CUDA_CHECK(cudaEventCreateWithFlags(&buf.done, cudaEventDisableTiming));
    if (buf.capacity < total) {
        if (buf.host) SFB_CUDA_CHECK(cudaFreeHost(buf.host));
        buf.host = nullptr;
        buf.capacity = std::max<int64_t>(total, std::max<int64_t>(4096, 2 * buf.capacity));
        SFB_CUDA_CHECK(cudaMallocHost(&buf.host, (size_t)buf.capacity * sizeof(int2)));
    }
    int64_t at = 0;
    for (auto& kv : bm->requests) {
        Request& r = kv.second;
        if (r.row < 0) continue;
        const int64_t base = r.row * bm->max_blocks;
        for (int64_t c = r.dirty_lo; c < (int64_t)r.table.size(); ++c) buf.host[at++] = make_int2((int)(base + c), r.table[(size_t)c]);
        r.dirty_lo = (int64_t)r.table.size();
    }
    table_scatter_kernel<<<(unsigned)ceil_div(total, (int64_t)256), 256, 0, st>>>(buf.host, total, bm->d_tables);
    SFB_CUDA_CHECK(cudaGetLastError());
    SFB_CUDA_CHECK(cudaEventRecord(buf.done, st));
    return total;
}

}  // extern "C"
