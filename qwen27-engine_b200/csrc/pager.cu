// Page bookkeeping for the paged q8_0 cache of q27b_attn_decode_paged / q27b_attn_prep_paged: which pool
// pages back which positions of which sequence. Host code only; the tables it produces are what those
// operators read on the device.
//
// The reference keeps one contiguous cache per sequence and relies on one property of it when the server
// reuses a prompt prefix: "KV rows below a position stay valid when the sequence is cut back to it"
// (src/model.h:177-180; Engine::prepare, src/engine.cpp:228-291, cuts the live sequence back to the
// longest common prefix and reads on from there). Here that is q27b_pager_cut: the pages that hold rows
// below the new length stay where they are, the others go back to the pool. q27b_pager_fork is what a page
// table adds: a second sequence that starts as a prefix of another shares the full pages of that prefix
// instead of copying them (reference counts); only a partly filled last page has to be copied, and the
// call says which.
#include "common.cuh"
#include "host.h"

#include <exception>
#include <mutex>
#include <vector>

namespace q27b {
namespace {

struct Seq {
  bool open = false;
  int len = 0;
  std::vector<int> pages;  // page j backs positions 256 j .. 256 j + 255
};

}  // namespace
}  // namespace q27b

struct q27b_pager {
  int n_pages, max_seqs, max_pages;
  std::vector<int> refs;       // per page: sequences that hold it
  std::vector<int> free_list;  // pages with refs == 0, taken from the back
  std::vector<q27b::Seq> seqs;
  std::mutex mu;
};

using namespace q27b;

namespace {

int pages_for(int len) { return (len + Q27B_PAGE - 1) / Q27B_PAGE; }

void drop_page(q27b_pager* pg, int page) {
  if (--pg->refs[page] == 0) pg->free_list.push_back(page);
}

Seq* seq_of(q27b_pager* pg, int seq) {
  if (seq < 0 || seq >= pg->max_seqs || !pg->seqs[seq].open) return nullptr;
  return &pg->seqs[seq];
}

}  // namespace

extern "C" {

int q27b_pager_create(int n_pages, int max_seqs, int max_pages_per_seq, q27b_pager** out) {
  if (!out || n_pages < 1 || max_seqs < 1 || max_pages_per_seq < 1) return fail(Q27B_BAD_SHAPE, "pager_create: bad shape");
  q27b_pager* pg = nullptr;
  try {  // (no exception crosses the C boundary)
    pg = new q27b_pager;
    pg->n_pages = n_pages;
    pg->max_seqs = max_seqs;
    pg->max_pages = max_pages_per_seq;
    pg->refs.assign(n_pages, 0);
    pg->free_list.resize(n_pages);
    for (int i = 0; i < n_pages; i++) pg->free_list[i] = n_pages - 1 - i;  // page 0 is handed out first
    pg->seqs.resize(max_seqs);
    for (auto& q : pg->seqs) q.pages.reserve(max_pages_per_seq);  // extend and fork then never allocate
  } catch (const std::exception&) {
    delete pg;
    return fail(Q27B_UNSUPPORTED, "pager_create: out of host memory");
  }
  *out = pg;
  return Q27B_OK;
}

void q27b_pager_destroy(q27b_pager* pg) { delete pg; }

int q27b_pager_open(q27b_pager* pg, int* seq) {
  if (!pg || !seq) return fail(Q27B_BAD_SHAPE, "pager_open: null pointer");
  std::lock_guard<std::mutex> lock(pg->mu);
  for (int i = 0; i < pg->max_seqs; i++)
    if (!pg->seqs[i].open) {
      pg->seqs[i].open = true;
      pg->seqs[i].len = 0;
      pg->seqs[i].pages.clear();
      *seq = i;
      return Q27B_OK;
    }
  return fail(Q27B_UNSUPPORTED, "pager_open: all sequence slots are in use");
}

int q27b_pager_extend(q27b_pager* pg, int seq, int new_len) {
  if (!pg) return fail(Q27B_BAD_SHAPE, "pager_extend: null pointer");
  std::lock_guard<std::mutex> lock(pg->mu);
  Seq* s = seq_of(pg, seq);
  if (!s) return fail(Q27B_BAD_SHAPE, "pager_extend: no such sequence");
  if (new_len < s->len || pages_for(new_len) > pg->max_pages) return fail(Q27B_BAD_SHAPE, "pager_extend: bad length");
  const int have = (int)s->pages.size(), need = pages_for(new_len);
  // A shared last page that is only partly filled cannot take this sequence's new rows.
  if (new_len > s->len && s->len % Q27B_PAGE != 0 && pg->refs[s->pages[have - 1]] > 1)
    return fail(Q27B_UNSUPPORTED, "pager_extend: the last page is shared and not full (fork copies it first)");
  if (need - have > (int)pg->free_list.size())
    return fail(Q27B_UNSUPPORTED, "pager_extend: the pool has no free pages left");  // nothing changed
  for (int j = have; j < need; j++) {
    const int page = pg->free_list.back();
    pg->free_list.pop_back();
    pg->refs[page] = 1;
    s->pages.push_back(page);
  }
  s->len = new_len;
  return Q27B_OK;
}

int q27b_pager_cut(q27b_pager* pg, int seq, int new_len) {
  if (!pg) return fail(Q27B_BAD_SHAPE, "pager_cut: null pointer");
  std::lock_guard<std::mutex> lock(pg->mu);
  Seq* s = seq_of(pg, seq);
  if (!s) return fail(Q27B_BAD_SHAPE, "pager_cut: no such sequence");
  if (new_len < 0 || new_len > s->len) return fail(Q27B_BAD_SHAPE, "pager_cut: bad length");
  const int keep = pages_for(new_len);
  while ((int)s->pages.size() > keep) {
    drop_page(pg, s->pages.back());
    s->pages.pop_back();
  }
  s->len = new_len;
  return Q27B_OK;
}

int q27b_pager_close(q27b_pager* pg, int seq) {
  if (!pg) return fail(Q27B_BAD_SHAPE, "pager_close: null pointer");
  std::lock_guard<std::mutex> lock(pg->mu);
  Seq* s = seq_of(pg, seq);
  if (!s) return fail(Q27B_BAD_SHAPE, "pager_close: no such sequence");
  for (int page : s->pages) drop_page(pg, page);
  s->pages.clear();
  s->len = 0;
  s->open = false;
  return Q27B_OK;
}

int q27b_pager_fork(q27b_pager* pg, int seq, int prefix_len, int* new_seq, int* copy_src_page, int* copy_dst_page,
                    int* copy_rows) {
  if (!pg || !new_seq || !copy_src_page || !copy_dst_page || !copy_rows) return fail(Q27B_BAD_SHAPE, "pager_fork: null pointer");
  std::lock_guard<std::mutex> lock(pg->mu);
  Seq* s = seq_of(pg, seq);
  if (!s) return fail(Q27B_BAD_SHAPE, "pager_fork: no such sequence");
  if (prefix_len < 0 || prefix_len > s->len) return fail(Q27B_BAD_SHAPE, "pager_fork: bad length");
  int slot = -1;
  for (int i = 0; i < pg->max_seqs && slot < 0; i++)
    if (!pg->seqs[i].open) slot = i;
  if (slot < 0) return fail(Q27B_UNSUPPORTED, "pager_fork: all sequence slots are in use");
  const int full = prefix_len / Q27B_PAGE, rest = prefix_len % Q27B_PAGE;
  if (rest && pg->free_list.empty()) return fail(Q27B_UNSUPPORTED, "pager_fork: the pool has no free pages left");
  Seq* d = &pg->seqs[slot];
  s = &pg->seqs[seq];
  d->open = true;
  d->len = prefix_len;
  d->pages.assign(s->pages.begin(), s->pages.begin() + full);
  for (int page : d->pages) pg->refs[page]++;
  *copy_src_page = *copy_dst_page = -1;
  *copy_rows = 0;
  if (rest) {  // the partly filled page gets a copy of its own: both sequences will write behind the prefix
    const int page = pg->free_list.back();
    pg->free_list.pop_back();
    pg->refs[page] = 1;
    d->pages.push_back(page);
    *copy_src_page = s->pages[full];
    *copy_dst_page = page;
    *copy_rows = rest;
  }
  *new_seq = slot;
  return Q27B_OK;
}

int q27b_pager_unshare(q27b_pager* pg, int seq, int* copy_src_page, int* copy_dst_page, int* copy_rows) {
  if (!pg || !copy_src_page || !copy_dst_page || !copy_rows) return fail(Q27B_BAD_SHAPE, "pager_unshare: null pointer");
  std::lock_guard<std::mutex> lock(pg->mu);
  Seq* s = seq_of(pg, seq);
  if (!s) return fail(Q27B_BAD_SHAPE, "pager_unshare: no such sequence");
  *copy_src_page = *copy_dst_page = -1;
  *copy_rows = 0;
  const int rest = s->len % Q27B_PAGE;
  if (!rest || pg->refs[s->pages.back()] == 1) return Q27B_OK;  // nothing to do
  if (pg->free_list.empty()) return fail(Q27B_UNSUPPORTED, "pager_unshare: the pool has no free pages left");
  const int page = pg->free_list.back();
  pg->free_list.pop_back();
  pg->refs[page] = 1;
  *copy_src_page = s->pages.back();
  *copy_dst_page = page;
  *copy_rows = rest;
  pg->refs[s->pages.back()]--;  // still held by somebody else
  s->pages.back() = page;
  return Q27B_OK;
}

int q27b_kv_page_copy(void* pool, int src_page, int dst_page, int rows, int nkvh, int n_pages, void* stream) {
  if (!pool || nkvh < 1 || n_pages < 1 || src_page < 0 || src_page >= n_pages || dst_page < 0 || dst_page >= n_pages ||
      src_page == dst_page || rows < 1 || rows > Q27B_PAGE)
    return fail(Q27B_BAD_SHAPE, "kv_page_copy: bad argument");
  uint8_t* vals = (uint8_t*)pool;
  uint8_t* scales = vals + (size_t)n_pages * nkvh * Q27B_PAGE * AD;
  for (int h = 0; h < nkvh; h++) {  // per head the first `rows` rows of a page are contiguous: values, then scales
    const size_t s = ((size_t)src_page * nkvh + h) * Q27B_PAGE, d = ((size_t)dst_page * nkvh + h) * Q27B_PAGE;
    Q27B_CK(cudaMemcpyAsync(vals + d * AD, vals + s * AD, (size_t)rows * AD, cudaMemcpyDeviceToDevice, (cudaStream_t)stream));
    Q27B_CK(cudaMemcpyAsync(scales + d * 16, scales + s * 16, (size_t)rows * 16, cudaMemcpyDeviceToDevice, (cudaStream_t)stream));
  }
  return Q27B_OK;
}

int q27b_pager_free_pages(q27b_pager* pg) {
  if (!pg) return -1;
  std::lock_guard<std::mutex> lock(pg->mu);
  return (int)pg->free_list.size();
}

int q27b_pager_len(q27b_pager* pg, int seq) {
  if (!pg) return -1;
  std::lock_guard<std::mutex> lock(pg->mu);
  Seq* s = seq_of(pg, seq);
  return s ? s->len : -1;
}

int q27b_pager_tables(q27b_pager* pg, const int* seqs, int B, int* page_table, int* seq_len) {
  if (!pg || !seqs || !page_table || !seq_len || B < 1) return fail(Q27B_BAD_SHAPE, "pager_tables: bad argument");
  std::lock_guard<std::mutex> lock(pg->mu);
  for (int b = 0; b < B; b++) {
    Seq* s = seq_of(pg, seqs[b]);
    if (!s) return fail(Q27B_BAD_SHAPE, "pager_tables: no such sequence");
    int* row = page_table + (size_t)b * pg->max_pages;
    for (int j = 0; j < pg->max_pages; j++) row[j] = j < (int)s->pages.size() ? s->pages[j] : -1;
    seq_len[b] = s->len;
  }
  return Q27B_OK;
}

}  // extern "C"
