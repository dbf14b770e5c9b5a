// Host-side runtime pieces with a plain C interface (loaded with ctypes; no Python or torch headers):
//
//   * the "world" tokenizer's greedy longest-match encoder over a byte trie, one document or a batch of
//     documents spread over threads (corpus conversion is dominated by this loop);
//   * the batch gather of the data loader: `rows` windows of `window` tokens read from the memory-mapped
//     token stream (uint8 / uint16 / int32 / int64 ... storage) into the int32 input / target matrices of a
//     training batch, written straight into caller-provided (pinned) buffers, spread over threads.
//
// Every entry point validates its arguments and returns a negative code instead of touching memory it was
// not given; nothing here allocates on behalf of the caller except the tokenizer handle.

#include <algorithm>
#include <cstdint>
#include <cstring>
#include <new>
#include <thread>
#include <vector>

namespace {

// Byte trie stored as flat arrays.  Node 0 is the root.  The children of a node are a sorted run of
// (byte, child) pairs in `edge_byte` / `edge_child`; the root has a direct 256-entry table because every
// lookup starts there.  `token_of[node]` is the token id that ends at the node, or -1.
struct Trie {
  std::vector<int32_t> first_edge;   // per node: index of its first edge
  std::vector<int32_t> edge_count;   // per node
  std::vector<uint8_t> edge_byte;
  std::vector<int32_t> edge_child;
  std::vector<int32_t> token_of;
  int32_t root_child[256];
  int32_t max_token_len = 0;

  int32_t child(int32_t node, uint8_t byte) const {
    if (node == 0) return root_child[byte];
    const int32_t lo = first_edge[node], n = edge_count[node];
    const uint8_t* b = edge_byte.data() + lo;
    if (n <= 8) {
      for (int32_t i = 0; i < n; ++i)
        if (b[i] == byte) return edge_child[lo + i];
      return -1;
    }
    const uint8_t* e = std::lower_bound(b, b + n, byte);
    return (e != b + n && *e == byte) ? edge_child[lo + int32_t(e - b)] : -1;
  }
};

struct BuildNode {
  std::vector<std::pair<uint8_t, int32_t>> kids;
  int32_t token = -1;
};

Trie* build_trie(const uint8_t* blob, const int64_t* offsets, const int32_t* ids, int32_t n_tokens) {
  std::vector<BuildNode> nodes(1);
  int32_t max_len = 0;
  for (int32_t t = 0; t < n_tokens; ++t) {
    const int64_t b = offsets[t], e = offsets[t + 1];
    if (e < b) return nullptr;
    if (e == b) continue;   // the empty byte string matches nothing
    max_len = std::max<int32_t>(max_len, int32_t(e - b));
    int32_t cur = 0;
    for (int64_t i = b; i < e; ++i) {
      const uint8_t c = blob[i];
      int32_t next = -1;
      for (auto& kv : nodes[cur].kids)
        if (kv.first == c) { next = kv.second; break; }
      if (next < 0) {
        next = int32_t(nodes.size());
        nodes[cur].kids.emplace_back(c, next);
        nodes.emplace_back();
      }
      cur = next;
    }
    nodes[cur].token = ids[t];   // a repeated byte string keeps the last id, as a dictionary would
  }
  Trie* tr = new (std::nothrow) Trie();
  if (tr == nullptr) return nullptr;
  const size_t n = nodes.size();
  tr->first_edge.resize(n);
  tr->edge_count.resize(n);
  tr->token_of.resize(n);
  tr->max_token_len = max_len;
  std::fill(tr->root_child, tr->root_child + 256, -1);
  size_t total_edges = 0;
  for (auto& nd : nodes) total_edges += nd.kids.size();
  tr->edge_byte.reserve(total_edges);
  tr->edge_child.reserve(total_edges);
  for (size_t i = 0; i < n; ++i) {
    auto& kids = nodes[i].kids;
    std::sort(kids.begin(), kids.end());
    tr->first_edge[i] = int32_t(tr->edge_byte.size());
    tr->edge_count[i] = int32_t(kids.size());
    tr->token_of[i] = nodes[i].token;
    for (auto& kv : kids) {
      tr->edge_byte.push_back(kv.first);
      tr->edge_child.push_back(kv.second);
      if (i == 0) tr->root_child[kv.first] = kv.second;
    }
  }
  return tr;
}

// Greedy longest match.  Returns the number of ids written, -(pos + 1) when the byte at `pos` starts no
// vocabulary entry, or INT64_MIN when `out` is too small.
int64_t encode_one(const Trie& tr, const uint8_t* src, int64_t n, int32_t* out, int64_t cap) {
  int64_t pos = 0, count = 0;
  while (pos < n) {
    int32_t node = 0, best = -1;
    int64_t best_end = pos;
    for (int64_t i = pos; i < n; ++i) {
      node = tr.child(node, src[i]);
      if (node < 0) break;
      const int32_t tok = tr.token_of[node];
      if (tok >= 0) { best = tok; best_end = i + 1; }
    }
    if (best < 0) return -(pos + 1);
    if (count >= cap) return INT64_MIN;
    out[count++] = best;
    pos = best_end;
  }
  return count;
}

template <typename T>
void gather_rows_typed(const T* base, int64_t total, const int64_t* offsets, int64_t row_begin, int64_t row_end,
                       int64_t window, int32_t* inputs, int32_t* targets) {
  const int64_t ctx = window - 1;
  for (int64_t r = row_begin; r < row_end; ++r) {
    const T* src = base + offsets[r];
    int32_t* in = inputs + r * ctx;
    int32_t* tg = targets + r * ctx;
    (void)total;
    int32_t prev = int32_t(src[0]);
    for (int64_t j = 1; j < window; ++j) {
      const int32_t cur = int32_t(src[j]);
      in[j - 1] = prev;
      tg[j - 1] = cur;
      prev = cur;
    }
  }
}

int clamp_threads(int threads, int64_t items) {
  if (threads <= 0) threads = int(std::thread::hardware_concurrency());
  if (threads <= 0) threads = 1;
  if (int64_t(threads) > items) threads = int(std::max<int64_t>(items, 1));
  return std::min(threads, 64);
}

}  // namespace

extern "C" {

// `blob` holds the token byte strings back to back; token t is blob[offsets[t] .. offsets[t + 1]) with id ids[t].
void* rk_tok_create(const uint8_t* blob, const int64_t* offsets, const int32_t* ids, int32_t n_tokens) {
  if (blob == nullptr || offsets == nullptr || ids == nullptr || n_tokens <= 0) return nullptr;
  return build_trie(blob, offsets, ids, n_tokens);
}

void rk_tok_free(void* handle) { delete static_cast<Trie*>(handle); }

int32_t rk_tok_max_token_len(const void* handle) {
  return handle == nullptr ? -1 : static_cast<const Trie*>(handle)->max_token_len;
}

int64_t rk_tok_node_count(const void* handle) {
  return handle == nullptr ? -1 : int64_t(static_cast<const Trie*>(handle)->token_of.size());
}

int64_t rk_tok_encode(const void* handle, const uint8_t* src, int64_t n, int32_t* out, int64_t cap) {
  if (handle == nullptr || n < 0 || cap < 0 || (n > 0 && src == nullptr) || (cap > 0 && out == nullptr)) return INT64_MIN;
  return encode_one(*static_cast<const Trie*>(handle), src, n, out, cap);
}

// Documents d = 0 .. n_docs-1 are src[doc_offsets[d] .. doc_offsets[d + 1]); the ids of document d go to
// out[out_offsets[d] ..) with room for out_offsets[d + 1] - out_offsets[d] ids (a document never yields more ids than it
// has bytes).  counts[d] receives the result of the single-document call.  Returns 0, or -1 on bad arguments.
int32_t rk_tok_encode_batch(const void* handle, const uint8_t* src, const int64_t* doc_offsets, int64_t n_docs, int32_t* out,
                            const int64_t* out_offsets, int64_t* counts, int32_t threads) {
  if (handle == nullptr || doc_offsets == nullptr || out_offsets == nullptr || counts == nullptr || n_docs < 0) return -1;
  if (n_docs == 0) return 0;
  if (src == nullptr || out == nullptr) return -1;
  const Trie& tr = *static_cast<const Trie*>(handle);
  const int nt = clamp_threads(threads, n_docs);
  auto work = [&](int64_t lo, int64_t hi) {
    for (int64_t d = lo; d < hi; ++d) {
      const int64_t n = doc_offsets[d + 1] - doc_offsets[d], cap = out_offsets[d + 1] - out_offsets[d];
      counts[d] = (n < 0 || cap < 0) ? INT64_MIN : encode_one(tr, src + doc_offsets[d], n, out + out_offsets[d], cap);
    }
  };
  if (nt == 1) { work(0, n_docs); return 0; }
  std::vector<std::thread> pool;
  const int64_t per = (n_docs + nt - 1) / nt;
  for (int t = 0; t < nt; ++t) {
    const int64_t lo = t * per, hi = std::min<int64_t>(n_docs, lo + per);
    if (lo < hi) pool.emplace_back(work, lo, hi);
  }
  for (auto& th : pool) th.join();
  return 0;
}

// Rows r = 0 .. rows-1: tokens base[offsets[r] .. offsets[r] + window) of a stream of `total` elements of `elem_size`
// bytes (signedness as given); inputs[r] = the first window-1 of them, targets[r] = the last window-1, both int32,
// row-major [rows, window-1].  Returns 0, -1 on bad arguments, -2 when a window leaves the stream.
int32_t rk_gather_rows(const void* base, int32_t elem_size, int32_t is_signed, int64_t total, const int64_t* offsets,
                       int64_t rows, int64_t window, int32_t* inputs, int32_t* targets, int32_t threads) {
  if (base == nullptr || offsets == nullptr || inputs == nullptr || targets == nullptr || rows < 0 || window < 2 || total < 0)
    return -1;
  if (elem_size != 1 && elem_size != 2 && elem_size != 4 && elem_size != 8) return -1;
  for (int64_t r = 0; r < rows; ++r)
    if (offsets[r] < 0 || offsets[r] + window > total) return -2;
  if (rows == 0) return 0;
  const int nt = clamp_threads(threads, rows);
  auto work = [&](int64_t lo, int64_t hi) {
    switch (elem_size * 2 + (is_signed ? 1 : 0)) {
      case 2: gather_rows_typed(static_cast<const uint8_t*>(base), total, offsets, lo, hi, window, inputs, targets); break;
      case 3: gather_rows_typed(static_cast<const int8_t*>(base), total, offsets, lo, hi, window, inputs, targets); break;
      case 4: gather_rows_typed(static_cast<const uint16_t*>(base), total, offsets, lo, hi, window, inputs, targets); break;
      case 5: gather_rows_typed(static_cast<const int16_t*>(base), total, offsets, lo, hi, window, inputs, targets); break;
      case 8: gather_rows_typed(static_cast<const uint32_t*>(base), total, offsets, lo, hi, window, inputs, targets); break;
      case 9: gather_rows_typed(static_cast<const int32_t*>(base), total, offsets, lo, hi, window, inputs, targets); break;
      case 16: gather_rows_typed(static_cast<const uint64_t*>(base), total, offsets, lo, hi, window, inputs, targets); break;
      default: gather_rows_typed(static_cast<const int64_t*>(base), total, offsets, lo, hi, window, inputs, targets); break;
    }
  };
  if (nt == 1) { work(0, rows); return 0; }
  std::vector<std::thread> pool;
  const int64_t per = (rows + nt - 1) / nt;
  for (int t = 0; t < nt; ++t) {
    const int64_t lo = t * per, hi = std::min<int64_t>(rows, lo + per);
    if (lo < hi) pool.emplace_back(work, lo, hi);
  }
  for (auto& th : pool) th.join();
  return 0;
}

int32_t rk_host_runtime_version() { return 1; }

}  // extern "C"
