// Native host runtime: the per-request / per-step bookkeeping that sits on the engine thread's critical path.
//   BlockPool   ref-counted KV blocks, LIFO free lists, fast tier before slow tier
//   RadixCache  compressed radix tree over whole blocks of token ids (match + lock, insert, LRU eviction)
//   table_slots flat KV cell index of every position of a step (block table -> slots)
//   pack_decode the packed int32 input record of a CUDA-graph decode step
// Semantics are those of the Python classes in legion_b200/kv (which remain as the fallback and the executable
// specification: tests/test_kv.py runs both). Counterparts in the reference: src/kv/blocks.rs, src/kv/radix.rs.
#include <pybind11/numpy.h>
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include <algorithm>
#include <cstdint>
#include <cstring>
#include <map>
#include <memory>
#include <stdexcept>
#include <string>
#include <unordered_map>
#include <vector>

namespace py = pybind11;

// The exception type raised when the pool runs dry is the Python package's own class (installed once at import by
// legion_b200.kv.blocks), so `except OutOfBlocks` matches whichever implementation backs the pool.
static py::object& oob_type() {
  static py::object* t = new py::object(py::reinterpret_borrow<py::object>(PyExc_RuntimeError));
  return *t;
}
[[noreturn]] static void throw_assert(const char* msg) {
  PyErr_SetString(PyExc_AssertionError, msg);
  throw py::error_already_set();
}
[[noreturn]] static void throw_out_of_blocks(const std::string& msg) {
  PyErr_SetString(oob_type().ptr(), msg.c_str());
  throw py::error_already_set();
}

class BlockPool {
 public:
  BlockPool(int n_blocks, int block_size, int n_slow)
      : block_size(block_size), n_blocks(n_blocks), n_slow(n_slow), ref_(size_t(n_blocks + n_slow), 0) {
    for (int b = n_blocks - 1; b >= 0; --b) free_fast_.push_back(b);
    for (int b = n_blocks + n_slow - 1; b >= n_blocks; --b) free_slow_.push_back(b);
  }
  int free_count() const { return int(free_fast_.size() + free_slow_.size()); }
  int free_fast() const { return int(free_fast_.size()); }
  int used() const { return n_blocks + n_slow - free_count(); }
  int total() const { return n_blocks + n_slow; }
  int refcount(int b) const { return ref_.at(size_t(b)); }
  bool is_slow(int b) const { return b >= n_blocks; }
  int blocks_for(long n_tokens) const { return int((n_tokens + block_size - 1) / block_size); }

  std::vector<int> alloc(int n, bool allow_slow) {
    const int avail = int(free_fast_.size()) + (allow_slow ? int(free_slow_.size()) : 0);
    if (n > avail) throw_out_of_blocks("need " + std::to_string(n) + " blocks, " + std::to_string(avail) + " free");
    std::vector<int> out;
    out.reserve(size_t(n));
    for (int i = 0; i < n; ++i) {
      int b;
      if (!free_fast_.empty()) { b = free_fast_.back(); free_fast_.pop_back(); }
      else { b = free_slow_.back(); free_slow_.pop_back(); }
      ref_[size_t(b)] = 1;
      out.push_back(b);
    }
    return out;
  }
  void incref(int b) {
    if (b < 0 || b >= total() || ref_[size_t(b)] <= 0) throw_assert("incref of a free block");
    ++ref_[size_t(b)];
  }
  void decref(int b) {
    if (b < 0 || b >= total() || ref_[size_t(b)] <= 0) throw_assert("decref of a free block");
    if (--ref_[size_t(b)] == 0) (is_slow(b) ? free_slow_ : free_fast_).push_back(b);
  }
  void release(const std::vector<int>& blocks) {
    for (auto it = blocks.rbegin(); it != blocks.rend(); ++it) decref(*it);
  }

  const int block_size, n_blocks, n_slow;

 private:
  std::vector<int> ref_, free_fast_, free_slow_;
};

// ---------------------------------------------------------------------------------------------------
struct Node {
  std::vector<int> key;       // token ids of this edge (len = blocks.size() * bs)
  std::vector<int> blocks;
  std::map<std::vector<int>, Node*> children;   // keyed by the first block's tokens
  Node* parent = nullptr;
  int locks = 0;
  long tick = 0;
  long id = 0;
};

class RadixCache {
 public:
  explicit RadixCache(std::shared_ptr<BlockPool> pool) : pool_(std::move(pool)), bs_(pool_->block_size) {
    root_ = make_node();
  }
  ~RadixCache() {
    for (auto& kv : nodes_) delete kv.second;
  }

  // returns (blocks, n_tokens, handle); handle 0 = nothing locked
  py::tuple match_prefix(const std::vector<int>& tokens, bool lock, py::object max_tokens) {
    long limit = long(tokens.size());
    if (!max_tokens.is_none()) limit = std::min<long>(limit, max_tokens.cast<long>());
    Node* node = root_;
    long off = 0;
    std::vector<int> blocks;
    while (off + bs_ <= limit) {
      auto it = node->children.find(first(tokens, off));
      if (it == node->children.end()) break;
      Node* child = it->second;
      const int n_edge = int(child->blocks.size());
      int m = 0;
      while (m < n_edge && off + long(m + 1) * bs_ <= limit &&
             std::equal(tokens.begin() + off + long(m) * bs_, tokens.begin() + off + long(m + 1) * bs_,
                        child->key.begin() + long(m) * bs_))
        ++m;
      if (m == 0) break;
      if (m < n_edge) child = split(child, m);
      blocks.insert(blocks.end(), child->blocks.begin(), child->blocks.end());
      off += long(m) * bs_;
      node = child;
      touch(node);
      if (m < n_edge) break;
    }
    lookup_tokens += long(tokens.size());
    hit_tokens += off;
    long handle = 0;
    if (lock) {
      for (Node* n = node; n != nullptr; n = n->parent) ++n->locks;
      handle = node->id;
    }
    return py::make_tuple(blocks, off, lock ? py::cast(handle) : py::none());
  }

  void unlock(py::object handle) {
    if (handle.is_none()) return;
    auto it = nodes_.find(handle.cast<long>());
    if (it == nodes_.end()) throw_assert("unlock of an unknown radix handle");
    for (Node* n = it->second; n != nullptr; n = n->parent) {
      if (--n->locks < 0) throw_assert("radix lock count below zero");
    }
  }

  int insert(const std::vector<int>& tokens, const std::vector<int>& blocks) {
    const long n_full = std::min<long>(long(tokens.size()) / bs_, long(blocks.size()));
    Node* node = root_;
    long off = 0, i = 0;
    int adopted = 0;
    while (i < n_full) {
      auto key1 = first(tokens, off);
      auto it = node->children.find(key1);
      if (it == node->children.end()) {
        Node* nn = make_node();
        nn->key.assign(tokens.begin() + off, tokens.begin() + n_full * bs_);
        nn->blocks.assign(blocks.begin() + i, blocks.begin() + n_full);
        nn->parent = node;
        for (int b : nn->blocks) pool_->incref(b);
        adopted += int(nn->blocks.size());
        n_cached_blocks += long(nn->blocks.size());
        node->children[key1] = nn;
        touch(nn);
        return adopted;
      }
      Node* child = it->second;
      const int n_edge = int(child->blocks.size());
      int m = 0;
      while (m < n_edge && i + m < n_full &&
             std::equal(tokens.begin() + off + long(m) * bs_, tokens.begin() + off + long(m + 1) * bs_,
                        child->key.begin() + long(m) * bs_))
        ++m;
      if (m < n_edge) child = split(child, m);
      touch(child);
      node = child;
      off += long(m) * bs_;
      i += m;
    }
    return adopted;
  }

  // on_evict(prefix_tokens, block) is called for every block before it is released (None: no callback)
  int evict(int n_blocks, py::object on_evict) {
    int freed = 0;
    const bool cb = !on_evict.is_none();
    while (freed < n_blocks) {
      Node* leaf = nullptr;
      for (auto& kv : nodes_) {
        Node* n = kv.second;
        if (n == root_ || !n->children.empty() || n->locks != 0 || n->parent == nullptr) continue;
        if (leaf == nullptr || n->tick < leaf->tick) leaf = n;
      }
      if (leaf == nullptr) break;
      std::vector<int> path;
      if (cb) {
        std::vector<Node*> chain;
        for (Node* n = leaf; n != nullptr && n != root_; n = n->parent) chain.push_back(n);
        for (auto it = chain.rbegin(); it != chain.rend(); ++it) path.insert(path.end(), (*it)->key.begin(), (*it)->key.end());
      }
      while (!leaf->blocks.empty() && freed < n_blocks) {
        const int b = leaf->blocks.back();
        if (cb) {
          on_evict(path, b);
          path.resize(path.size() - size_t(bs_));
        }
        leaf->blocks.pop_back();
        leaf->key.resize(leaf->blocks.size() * size_t(bs_));
        pool_->decref(b);
        --n_cached_blocks;
        ++freed;
      }
      if (leaf->blocks.empty()) {
        Node* parent = leaf->parent;
        for (auto it = parent->children.begin(); it != parent->children.end(); ++it) {
          if (it->second == leaf) { parent->children.erase(it); break; }
        }
        nodes_.erase(leaf->id);
        delete leaf;
      }
    }
    return freed;
  }
  void clear() { evict(int(n_cached_blocks) + 1, py::none()); }

  long n_cached_blocks = 0, hit_tokens = 0, lookup_tokens = 0;
  std::shared_ptr<BlockPool> pool() const { return pool_; }
  int bs() const { return bs_; }

 private:
  Node* make_node() {
    Node* n = new Node();
    n->id = ++next_id_;
    nodes_[n->id] = n;
    return n;
  }
  void touch(Node* n) { n->tick = ++tick_; }
  std::vector<int> first(const std::vector<int>& t, long off) const {
    return std::vector<int>(t.begin() + off, t.begin() + std::min<long>(long(t.size()), off + bs_));
  }
  // splits node's edge after n_blocks blocks; returns the new upper node
  Node* split(Node* node, int n_blocks) {
    const long cut = long(n_blocks) * bs_;
    Node* upper = make_node();
    upper->key.assign(node->key.begin(), node->key.begin() + cut);
    upper->blocks.assign(node->blocks.begin(), node->blocks.begin() + n_blocks);
    upper->parent = node->parent;
    upper->locks = node->locks;
    upper->tick = node->tick;
    node->parent->children[first(node->key, 0)] = upper;
    node->key.erase(node->key.begin(), node->key.begin() + cut);
    node->blocks.erase(node->blocks.begin(), node->blocks.begin() + n_blocks);
    node->parent = upper;
    upper->children[first(node->key, 0)] = node;
    return upper;
  }

  std::shared_ptr<BlockPool> pool_;
  int bs_;
  Node* root_;
  long tick_ = 0, next_id_ = 0;
  std::unordered_map<long, Node*> nodes_;
};

// flat KV cell of positions [start, start + n) of a sequence
static py::array_t<int64_t> table_slots(const std::vector<int>& blocks, int block_size, long start, long n) {
  py::array_t<int64_t> out(n);
  auto* o = out.mutable_data();
  for (long p = start; p < start + n; ++p) {
    const long bi = p / block_size;
    if (bi >= long(blocks.size())) throw std::out_of_range("position beyond the block table");
    o[p - start] = int64_t(blocks[size_t(bi)]) * block_size + p % block_size;
  }
  return out;
}

// Packed input record of a CUDA-graph decode step (one token per sequence), int32 words:
// [slots as int64 (2 words each) | token ids | positions | cu_q | ctx_lens | state slots | block table B x W]
// Rows >= n (padding up to the bucket size B) read token 0 at position 0 with context length 1, write no KV cell
// (slot -1), use the spare state slot `pad_state` and an all-zero table row.
static void pack_decode(py::array_t<int32_t, py::array::c_style> buf, int B, int W, int block_size, int pad_state,
                        const std::vector<int>& tokens, const std::vector<long>& positions,
                        const std::vector<int>& state_slots, const std::vector<std::vector<int>>& tables) {
  const size_t n = tokens.size();
  if (positions.size() != n || state_slots.size() != n || tables.size() != n || n > size_t(B))
    throw std::invalid_argument("pack_decode: inconsistent row counts");
  const size_t total = size_t(2 * B + B + B + (B + 1) + B + B) + size_t(B) * size_t(W);
  if (size_t(buf.size()) < total) throw std::invalid_argument("pack_decode: buffer too small");
  int32_t* w = buf.mutable_data();
  auto* slots = reinterpret_cast<int64_t*>(w);
  int32_t* tok = w + 2 * B;
  int32_t* pos = tok + B;
  int32_t* cu = pos + B;
  int32_t* ctx = cu + B + 1;
  int32_t* st = ctx + B;
  int32_t* bt = st + B;
  std::memset(bt, 0, sizeof(int32_t) * size_t(B) * size_t(W));
  for (int i = 0; i <= B; ++i) cu[i] = i;
  for (size_t i = 0; i < size_t(B); ++i) {
    if (i < n) {
      const long p = positions[i];
      const auto& t = tables[i];
      const long bi = p / block_size;
      if (bi >= long(t.size()) || long(t.size()) > W) throw std::out_of_range("pack_decode: block table");
      slots[i] = int64_t(t[size_t(bi)]) * block_size + p % block_size;
      tok[i] = tokens[i];
      pos[i] = int32_t(p);
      ctx[i] = int32_t(p + 1);
      st[i] = state_slots[i];
      std::copy(t.begin(), t.end(), bt + i * size_t(W));
    } else {
      slots[i] = -1;
      tok[i] = 0;
      pos[i] = 0;
      ctx[i] = 1;
      st[i] = pad_state;
    }
  }
}

// Byte-pair merges of one pre-tokenised word (byte-to-unicode mapped text): lowest-rank adjacent pair first, until no
// pair has a rank; pieces that are not in the vocabulary fall back to their single symbols.
// Same procedure as BpeTokenizer._bpe in legion_b200/loaders/tokenizer.py (reference: src/tokenizer/bpe.rs).
class BpeMerger {
 public:
  BpeMerger(const std::vector<std::string>& tokens, const std::vector<std::pair<std::string, std::string>>& merges) {
    vocab_.reserve(tokens.size() * 2);
    for (size_t i = 0; i < tokens.size(); ++i) vocab_.emplace(tokens[i], int(i));
    ranks_.reserve(merges.size() * 2);
    for (size_t r = 0; r < merges.size(); ++r) ranks_.emplace(key(merges[r].first, merges[r].second), int(r));
  }

  std::vector<int> encode_word(const std::string& word) const {
    std::vector<std::string> parts;
    for (size_t i = 0; i < word.size();) {        // split into UTF-8 symbols
      const unsigned char c = static_cast<unsigned char>(word[i]);
      const size_t n = c < 0x80 ? 1 : (c >> 5) == 6 ? 2 : (c >> 4) == 14 ? 3 : 4;
      parts.emplace_back(word.substr(i, n));
      i += n;
    }
    while (parts.size() > 1) {
      int best = -1;
      size_t bi = 0;
      for (size_t i = 0; i + 1 < parts.size(); ++i) {
        auto it = ranks_.find(key(parts[i], parts[i + 1]));
        if (it != ranks_.end() && (best < 0 || it->second < best)) { best = it->second; bi = i; }
      }
      if (best < 0) break;
      parts[bi] += parts[bi + 1];
      parts.erase(parts.begin() + long(bi) + 1);
    }
    std::vector<int> ids;
    for (const auto& p : parts) {
      auto it = vocab_.find(p);
      if (it != vocab_.end()) { ids.push_back(it->second); continue; }
      for (size_t i = 0; i < p.size();) {
        const unsigned char c = static_cast<unsigned char>(p[i]);
        const size_t n = c < 0x80 ? 1 : (c >> 5) == 6 ? 2 : (c >> 4) == 14 ? 3 : 4;
        auto s = vocab_.find(p.substr(i, n));
        if (s != vocab_.end()) ids.push_back(s->second);
        i += n;
      }
    }
    return ids;
  }

  std::vector<int> encode_words(const std::vector<std::string>& words) const {
    std::vector<int> out;
    for (const auto& w : words) {
      auto ids = encode_word(w);
      out.insert(out.end(), ids.begin(), ids.end());
    }
    return out;
  }

  // Pre-tokens as raw UTF-8 bytes (the pieces the pre-tokeniser's pattern cut): the byte-to-unicode mapping and the
  // merges of every piece, ids concatenated. Runs without the interpreter lock, so the chunks of a long prompt encode
  // on several threads at once (the reference's parallel pre-tokenisation, src/tokenizer/parallel.rs).
  std::vector<int> encode_pieces(const std::vector<std::string>& pieces) const {
    static const std::vector<std::string> table = byte_table();
    std::vector<int> out;
    std::string word;
    for (const auto& p : pieces) {
      word.clear();
      for (unsigned char c : p) word += table[c];
      auto ids = encode_word(word);
      out.insert(out.end(), ids.begin(), ids.end());
    }
    return out;
  }

 private:
  // GPT-2's byte-to-unicode table: printable bytes stand for themselves, the others for code points from 256 up
  static std::vector<std::string> byte_table() {
    std::vector<int> cp(256, -1);
    auto keep = [&](int lo, int hi) { for (int b = lo; b <= hi; ++b) cp[b] = b; };
    keep(33, 126); keep(161, 172); keep(174, 255);
    int n = 0;
    for (int b = 0; b < 256; ++b)
      if (cp[b] < 0) cp[b] = 256 + n++;
    std::vector<std::string> t(256);
    for (int b = 0; b < 256; ++b) {
      const int c = cp[b];
      if (c < 0x80) t[b] = std::string(1, char(c));
      else t[b] = std::string{char(0xC0 | (c >> 6)), char(0x80 | (c & 0x3F))};
    }
    return t;
  }
  static std::string key(const std::string& a, const std::string& b) {
    std::string k;
    k.reserve(a.size() + b.size() + 1);
    k += a;
    k += ' ';            // byte-to-unicode mapped pieces never contain a plain space
    k += b;
    return k;
  }
  std::unordered_map<std::string, int> vocab_, ranks_;
};

PYBIND11_MODULE(_host, m) {
  m.doc() = "legion_b200 native host runtime (KV block pool, radix prefix cache, step packing)";
  m.def("set_out_of_blocks", [](py::object t) { oob_type() = std::move(t); });
  py::class_<BlockPool, std::shared_ptr<BlockPool>>(m, "BlockPool")
      .def(py::init<int, int, int>(), py::arg("n_blocks"), py::arg("block_size"), py::arg("n_slow") = 0)
      .def_readonly("block_size", &BlockPool::block_size)
      .def_readonly("n_blocks", &BlockPool::n_blocks)
      .def_readonly("n_slow", &BlockPool::n_slow)
      .def_property_readonly("free", &BlockPool::free_count)
      .def_property_readonly("free_fast", &BlockPool::free_fast)
      .def_property_readonly("used", &BlockPool::used)
      .def_property_readonly("total", &BlockPool::total)
      .def("refcount", &BlockPool::refcount)
      .def("is_slow", &BlockPool::is_slow)
      .def("blocks_for", &BlockPool::blocks_for)
      .def("alloc", &BlockPool::alloc, py::arg("n") = 1, py::arg("allow_slow") = true)
      .def("incref", &BlockPool::incref)
      .def("decref", &BlockPool::decref)
      .def("release", &BlockPool::release);
  py::class_<RadixCache>(m, "RadixCache")
      .def(py::init<std::shared_ptr<BlockPool>>())
      .def("match_prefix", &RadixCache::match_prefix, py::arg("tokens"), py::arg("lock") = true,
           py::arg("max_tokens") = py::none())
      .def("unlock", &RadixCache::unlock)
      .def("insert", &RadixCache::insert)
      .def("evict", &RadixCache::evict, py::arg("n_blocks"), py::arg("on_evict") = py::none())
      .def("clear", &RadixCache::clear)
      .def_readwrite("n_cached_blocks", &RadixCache::n_cached_blocks)
      .def_readwrite("hit_tokens", &RadixCache::hit_tokens)
      .def_readwrite("lookup_tokens", &RadixCache::lookup_tokens)
      .def_property_readonly("pool", &RadixCache::pool)
      .def_property_readonly("bs", &RadixCache::bs);
  py::class_<BpeMerger>(m, "BpeMerger")
      .def(py::init<const std::vector<std::string>&, const std::vector<std::pair<std::string, std::string>>&>())
      .def("encode_word", &BpeMerger::encode_word)
      .def("encode_words", &BpeMerger::encode_words)
      .def("encode_pieces", [](const BpeMerger& m, const std::vector<py::bytes>& pieces) {
        std::vector<std::string> raw;
        raw.reserve(pieces.size());
        for (const auto& b : pieces) raw.emplace_back(std::string(b));
        py::gil_scoped_release release;
        return m.encode_pieces(raw);
      });
  m.def("table_slots", &table_slots);
  m.def("pack_decode", &pack_decode);
}
