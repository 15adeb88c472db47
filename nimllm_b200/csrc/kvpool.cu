// kvpool.cu -- block manager of the paged KV cache.
//
// The reference keeps one [blockSize, D] buffer per (layer, KV head) for ONE conversation and, when
// a turn would not fit, throws the whole cache away (src/chat.nim:86-91: resetKvCache + history
// cleared).  With pages the cache is a pool of fixed-size pages shared by any number of sequences:
// a sequence holds as many pages as its length needs, a finished sequence gives them back, and a
// full pool refuses the one request that does not fit instead of resetting everybody.  This file
// is the bookkeeping: which page holds which rows of which sequence (the device table
// nimllm_attn_decode_paged and nimllm_rope_append_paged read), a free list, and the upload of the
// table rows that changed.  Host code only -- no kernel; with `on_device = 0` it touches no CUDA
// call at all (callers that own the page memory themselves, and tests without a GPU).
#include <vector>

#include "common.cuh"

struct nimllm_kvpool {
    int n_pages, page_rows, n_kv_head, head_dim, dtype, n_layer, max_seqs, max_pages;
    bool on_device;
    void *k_pages, *v_pages;             // [n_layer][n_pages][n_kv_head][page_rows][head_dim] each, or null
    int32_t *table_dev;                  // [max_seqs][max_pages] or null
    std::vector<int32_t> table;          // host copy; -1 = no page
    std::vector<int32_t> n_held;         // pages held per sequence
    std::vector<int32_t> rows;           // rows reserved per sequence
    std::vector<int32_t> free_list;      // stack of free pages
    std::vector<char> dirty;             // sequences whose table row changed since the last sync
};

using namespace nimllm;

extern "C" {

nimllm_kvpool *nimllm_kvpool_create(int n_layer, int n_pages, int page_rows, int n_kv_head, int head_dim, int dtype,
                                    int max_seqs, int max_pages_per_seq, int on_device) {
    int shift = 0;
    while ((1 << shift) < page_rows) shift++;
    if (n_layer <= 0 || n_pages <= 0 || page_rows <= 0 || (1 << shift) != page_rows || n_kv_head <= 0 || head_dim <= 0 ||
        head_dim % 8 != 0 || !dtype_ok(dtype) || max_seqs <= 0 || max_pages_per_seq <= 0) {
        set_error("kvpool_create: bad arguments (page_rows must be a power of two)");
        return nullptr;
    }
    nimllm_kvpool *p = new nimllm_kvpool();
    p->n_layer = n_layer; p->n_pages = n_pages; p->page_rows = page_rows; p->n_kv_head = n_kv_head; p->head_dim = head_dim;
    p->dtype = dtype; p->max_seqs = max_seqs; p->max_pages = max_pages_per_seq; p->on_device = on_device != 0;
    p->k_pages = p->v_pages = nullptr; p->table_dev = nullptr;
    p->table.assign((size_t)max_seqs * max_pages_per_seq, -1);
    p->n_held.assign(max_seqs, 0);
    p->rows.assign(max_seqs, 0);
    p->dirty.assign(max_seqs, 1);
    p->free_list.resize(n_pages);
    for (int i = 0; i < n_pages; i++) p->free_list[i] = n_pages - 1 - i;      // page 0 is handed out first
    if (p->on_device) {
        const size_t bytes = (size_t)n_layer * n_pages * n_kv_head * page_rows * head_dim * dtype_size(dtype);
        if (cudaMalloc(&p->k_pages, bytes) != cudaSuccess || cudaMalloc(&p->v_pages, bytes) != cudaSuccess ||
            cudaMalloc((void **)&p->table_dev, p->table.size() * sizeof(int32_t)) != cudaSuccess) {
            set_error("kvpool_create: cudaMalloc failed (%zu bytes per pool)", bytes);
            cudaFree(p->k_pages); cudaFree(p->v_pages); cudaFree(p->table_dev);
            delete p;
            return nullptr;
        }
        cudaMemset(p->k_pages, 0, bytes);
        cudaMemset(p->v_pages, 0, bytes);
        cudaMemcpy(p->table_dev, p->table.data(), p->table.size() * sizeof(int32_t), cudaMemcpyHostToDevice);
        std::fill(p->dirty.begin(), p->dirty.end(), 0);
    }
    return p;
}

void nimllm_kvpool_destroy(nimllm_kvpool *p) {
    if (!p) return;
    if (p->on_device) { cudaFree(p->k_pages); cudaFree(p->v_pages); cudaFree(p->table_dev); }
    delete p;
}

/* Makes sure sequence `seq` holds pages for rows 0 .. rows_total-1 (it never shrinks here).  All or
 * nothing: when the pool cannot cover the request nothing changes and NIMLLM_ERR_WORKSPACE comes back
 * -- the caller decides whom to evict (nimllm_kvpool_release), nobody else's cache is touched. */
int nimllm_kvpool_reserve(nimllm_kvpool *p, int seq, int rows_total) {
    if (!p || seq < 0 || seq >= p->max_seqs || rows_total < 0) return fail(NIMLLM_ERR_ARG, "kvpool_reserve: bad arguments");
    const int need = (rows_total + p->page_rows - 1) / p->page_rows;
    if (need > p->max_pages)
        return fail(NIMLLM_ERR_ARG, "kvpool_reserve: %d rows need %d pages, the table holds %d per sequence", rows_total, need, p->max_pages);
    const int extra = need - p->n_held[seq];
    if (extra > (int)p->free_list.size())
        return fail(NIMLLM_ERR_WORKSPACE, "kvpool_reserve: %d more pages wanted, %zu free", extra, p->free_list.size());
    for (int i = 0; i < extra; i++) {
        p->table[(size_t)seq * p->max_pages + p->n_held[seq]] = p->free_list.back();
        p->free_list.pop_back();
        p->n_held[seq]++;
    }
    if (extra > 0) p->dirty[seq] = 1;
    if (rows_total > p->rows[seq]) p->rows[seq] = rows_total;
    return NIMLLM_OK;
}

/* Gives all pages of a sequence back (its next reserve starts an empty sequence). */
int nimllm_kvpool_release(nimllm_kvpool *p, int seq) {
    if (!p || seq < 0 || seq >= p->max_seqs) return fail(NIMLLM_ERR_ARG, "kvpool_release: bad arguments");
    for (int i = p->n_held[seq] - 1; i >= 0; i--) {
        int32_t &e = p->table[(size_t)seq * p->max_pages + i];
        p->free_list.push_back(e);
        e = -1;
    }
    if (p->n_held[seq] > 0) p->dirty[seq] = 1;
    p->n_held[seq] = 0;
    p->rows[seq] = 0;
    return NIMLLM_OK;
}

/* Uploads the table rows that changed since the last call (one cudaMemcpyAsync per changed sequence,
 * from the pool's own host copy: call it before the launches that read the table, on their stream). */
int nimllm_kvpool_sync(nimllm_kvpool *p, void *stream) {
    if (!p) return fail(NIMLLM_ERR_ARG, "kvpool_sync: null pool");
    if (!p->on_device) { std::fill(p->dirty.begin(), p->dirty.end(), 0); return NIMLLM_OK; }
    for (int s = 0; s < p->max_seqs; s++)
        if (p->dirty[s]) {
            cudaError_t e = cudaMemcpyAsync(p->table_dev + (size_t)s * p->max_pages, p->table.data() + (size_t)s * p->max_pages,
                                            p->max_pages * sizeof(int32_t), cudaMemcpyHostToDevice, (cudaStream_t)stream);
            if (e != cudaSuccess) return fail(NIMLLM_ERR_CUDA, "kvpool_sync: %s", cudaGetErrorString(e));
            p->dirty[s] = 0;
        }
    return NIMLLM_OK;
}

int nimllm_kvpool_free_pages(const nimllm_kvpool *p) { return p ? (int)p->free_list.size() : -1; }
int nimllm_kvpool_seq_pages(const nimllm_kvpool *p, int seq) { return (p && seq >= 0 && seq < p->max_seqs) ? p->n_held[seq] : -1; }
int nimllm_kvpool_seq_rows(const nimllm_kvpool *p, int seq) { return (p && seq >= 0 && seq < p->max_seqs) ? p->rows[seq] : -1; }
const int32_t *nimllm_kvpool_table_host(const nimllm_kvpool *p) { return p ? p->table.data() : nullptr; }
const int32_t *nimllm_kvpool_table(const nimllm_kvpool *p, int first_seq) {
    return (p && p->table_dev && first_seq >= 0 && first_seq < p->max_seqs) ? p->table_dev + (size_t)first_seq * p->max_pages : nullptr;
}
static void *layer_pages(const nimllm_kvpool *p, void *base, int layer) {
    if (!p || !base || layer < 0 || layer >= p->n_layer) return nullptr;
    return (char *)base + (size_t)layer * p->n_pages * p->n_kv_head * p->page_rows * p->head_dim * dtype_size(p->dtype);
}
void *nimllm_kvpool_k(const nimllm_kvpool *p, int layer) { return p ? layer_pages(p, p->k_pages, layer) : nullptr; }
void *nimllm_kvpool_v(const nimllm_kvpool *p, int layer) { return p ? layer_pages(p, p->v_pages, layer) : nullptr; }

}  // extern "C"
