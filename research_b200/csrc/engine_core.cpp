// Host-side core of the inference engine (C++17, C ABI for ctypes):
//
//   BlockPool    fixed-size KV blocks with reference counts and an O(1) free list
//   PrefixIndex  two interchangeable prefix caches over the pool
//                  - hash chain (vLLM / nano-vllm style, one 64-bit chained hash per full block)
//                  - radix tree  (SGLang style, block-granular edges, node splitting, LRU
//                                 eviction of unlocked leaves)
//   EngineCore   sequence table, waiting/running queues, continuous-batching scheduler
//                (decode first, then admit under batch-size / token / block budgets),
//                preemption by recompute, and the per-step batch builder that writes token
//                ids, positions, slot mapping, block tables and sampling rows straight into
//                pinned host buffers.
//
// Behaviour it reproduces: rollouts/inference/scheduler.py:15-84 (policy),
// rollouts/inference/cache/paged.py:57-203 (block table + prefix hits),
// rollouts/inference/context.py:10-150 (slot mapping); the radix cache is only a stub in the
// reference (cache/radix.py:42) and is implemented here for real.
#include <algorithm>
#include <cstdint>
#include <cstring>
#include <deque>
#include <memory>
#include <unordered_map>
#include <vector>

namespace {

using i64 = long long;

inline uint64_t mix64(uint64_t z) {
  z += 0x9E3779B97F4A7C15ull;
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  return z ^ (z >> 31);
}
inline uint64_t hash_block(const int* tok, int n, uint64_t prefix) {
  uint64_t h = mix64(prefix ^ 0xA0761D6478BD642Full);
  for (int i = 0; i < n; ++i) h = mix64(h ^ (uint64_t)(uint32_t)tok[i] * 0xE7037ED1A0B428DBull);
  return h;
}

// ------------------------------------------------------------------------------------------
struct BlockPool {
  int num_blocks, block_size;
  std::vector<int> ref;          // users of the block (sequences + the radix tree)
  std::vector<int> prev, next;   // intrusive free list (index num_blocks is the sentinel)
  std::vector<char> in_free;
  int free_count = 0;

  BlockPool(int n, int bs) : num_blocks(n), block_size(bs), ref(n, 0), prev(n + 1), next(n + 1), in_free(n, 0) {
    prev[n] = next[n] = n;
    for (int i = 0; i < n; ++i) push_back(i);
  }
  void push_back(int b) {
    int s = num_blocks;
    prev[b] = prev[s]; next[b] = s; next[prev[s]] = b; prev[s] = b;
    in_free[b] = 1; ++free_count;
  }
  void unlink(int b) {
    next[prev[b]] = next[b]; prev[next[b]] = prev[b];
    in_free[b] = 0; --free_count;
  }
  int pop_front() {
    if (free_count == 0) return -1;
    int b = next[num_blocks];
    unlink(b);
    return b;
  }
};

// ------------------------------------------------------------------------------------------
struct RadixNode {
  RadixNode* parent = nullptr;
  std::unordered_map<uint64_t, RadixNode*> children;  // keyed by hash of the edge's first block
  std::vector<int> tokens;   // multiple of block_size
  std::vector<int> blocks;
  int lock = 0;              // sequences currently pinned through this node
  uint64_t last_access = 0;
};

struct KVManager {
  BlockPool pool;
  int mode;  // 0 none, 1 hash chain, 2 radix
  // hash chain
  std::unordered_map<uint64_t, int> hash_to_block;
  std::vector<uint64_t> block_hash;
  std::vector<char> block_hashed;
  std::vector<std::vector<int>> block_tokens;
  // radix
  RadixNode root;
  uint64_t clock = 0;
  i64 evictable_blocks = 0;
  // stats
  i64 hit_tokens = 0, miss_tokens = 0, evictions = 0;

  KVManager(int n, int bs, int m) : pool(n, bs), mode(m), block_hash(n, 0), block_hashed(n, 0), block_tokens(n) {}
  ~KVManager() { free_subtree(&root); }

  void free_subtree(RadixNode* n) {
    for (auto& kv : n->children) { free_subtree(kv.second); delete kv.second; }
    n->children.clear();
  }

  int num_free() const { return pool.free_count + (mode == 2 ? (int)evictable_blocks : 0); }

  // ---- fresh block (evicting cached content if needed) ----
  int take_block() {
    if (pool.free_count == 0 && mode == 2) evict(1);
    int b = pool.pop_front();
    if (b < 0) return -1;
    if (mode == 1 && block_hashed[b]) {  // lazily drop stale hash entry of a recycled block
      auto it = hash_to_block.find(block_hash[b]);
      if (it != hash_to_block.end() && it->second == b) hash_to_block.erase(it);
      block_hashed[b] = 0;
      block_tokens[b].clear();
      ++evictions;
    }
    pool.ref[b] = 1;
    return b;
  }
  void unref(int b) {
    if (--pool.ref[b] == 0) pool.push_back(b);
  }

  // ---- hash chain ----
  // Returns number of leading full blocks found in the cache; fills out blocks and bumps refs.
  int match_hash(const int* tok, int n_full, std::vector<int>& out, uint64_t& chain) {
    const int bs = pool.block_size;
    int matched = 0;
    chain = 0;
    for (int i = 0; i < n_full; ++i) {
      uint64_t h = hash_block(tok + i * bs, bs, chain);
      auto it = hash_to_block.find(h);
      if (it == hash_to_block.end()) break;
      int b = it->second;
      if ((int)block_tokens[b].size() != bs || std::memcmp(block_tokens[b].data(), tok + i * bs, bs * sizeof(int)) != 0) break;
      if (pool.ref[b] == 0) pool.unlink(b);
      ++pool.ref[b];
      out.push_back(b);
      chain = h;
      ++matched;
    }
    return matched;
  }
  void register_hash(int b, const int* tok, uint64_t prefix, uint64_t& out_hash) {
    const int bs = pool.block_size;
    out_hash = hash_block(tok, bs, prefix);
    if (block_hashed[b]) return;
    if (hash_to_block.find(out_hash) != hash_to_block.end()) return;  // an equal block is already published
    hash_to_block[out_hash] = b;
    block_hash[b] = out_hash;
    block_hashed[b] = 1;
    block_tokens[b].assign(tok, tok + bs);
  }

  // ---- radix ----
  uint64_t edge_key(const int* tok) const { return hash_block(tok, pool.block_size, 0x5151); }

  // Splits an edge after keep_blocks blocks. A NEW node takes the head of the edge and is
  // linked between the parent and `node`; `node` keeps its identity (and its children) as the
  // tail, so sequences that pinned `node` still unpin the whole path when they release it.
  RadixNode* split(RadixNode* node, int keep_blocks) {
    const int bs = pool.block_size;
    RadixNode* head = new RadixNode();
    head->parent = node->parent;
    head->tokens.assign(node->tokens.begin(), node->tokens.begin() + keep_blocks * bs);
    head->blocks.assign(node->blocks.begin(), node->blocks.begin() + keep_blocks);
    head->lock = node->lock;
    head->last_access = node->last_access;
    node->parent->children[edge_key(head->tokens.data())] = head;
    node->tokens.erase(node->tokens.begin(), node->tokens.begin() + keep_blocks * bs);
    node->blocks.erase(node->blocks.begin(), node->blocks.begin() + keep_blocks);
    node->parent = head;
    head->children[edge_key(node->tokens.data())] = node;
    return head;
  }

  // Walks the tree along tok (n_full blocks). Returns the deepest node fully matched (after
  // splitting a partially matched edge) and appends the matched blocks to out.
  RadixNode* match_radix(const int* tok, int n_full, std::vector<int>& out) {
    const int bs = pool.block_size;
    RadixNode* node = &root;
    int i = 0;
    ++clock;
    while (i < n_full) {
      auto it = node->children.find(edge_key(tok + i * bs));
      if (it == node->children.end()) break;
      RadixNode* child = it->second;
      const int edge_blocks = (int)child->blocks.size();
      int m = 0;
      while (m < edge_blocks && i + m < n_full &&
             std::memcmp(child->tokens.data() + m * bs, tok + (i + m) * bs, bs * sizeof(int)) == 0)
        ++m;
      if (m == 0) break;
      const bool partial = m < edge_blocks;
      if (partial) child = split(child, m);
      for (int j = 0; j < m; ++j) out.push_back(child->blocks[j]);
      child->last_access = clock;
      node = child;
      i += m;
      if (partial) break;
    }
    return node;
  }
  void lock_path(RadixNode* n, int delta) {
    for (; n != nullptr && n != &root; n = n->parent) {
      if (n->lock == 0 && delta > 0) evictable_blocks -= (i64)n->blocks.size();
      n->lock += delta;
      if (n->lock == 0 && delta < 0) evictable_blocks += (i64)n->blocks.size();
    }
  }
  // Inserts blocks for tok[0 : n_full*bs]; `blocks` are the sequence's blocks. Blocks that
  // become part of the tree get one extra reference held by the tree.
  void insert_radix(const int* tok, int n_full, const int* blocks) {
    const int bs = pool.block_size;
    std::vector<int> matched;
    RadixNode* node = match_radix(tok, n_full, matched);
    const int have = (int)matched.size();
    if (have >= n_full) return;
    RadixNode* leaf = new RadixNode();
    leaf->parent = node;
    leaf->tokens.assign(tok + have * bs, tok + n_full * bs);
    leaf->blocks.assign(blocks + have, blocks + n_full);
    leaf->last_access = clock;
    for (int b : leaf->blocks) ++pool.ref[b];
    node->children[edge_key(leaf->tokens.data())] = leaf;
    evictable_blocks += (i64)leaf->blocks.size();
  }
  void collect_leaves(RadixNode* n, std::vector<RadixNode*>& out) {
    if (n != &root && n->children.empty() && n->lock == 0) out.push_back(n);
    for (auto& kv : n->children) collect_leaves(kv.second, out);
  }
  // Frees at least `want` blocks by dropping least-recently-used unlocked leaves.
  int evict(int want) {
    int freed = 0;
    while (freed < want) {
      std::vector<RadixNode*> leaves;
      collect_leaves(&root, leaves);
      if (leaves.empty()) break;
      std::sort(leaves.begin(), leaves.end(), [](RadixNode* a, RadixNode* b) { return a->last_access < b->last_access; });
      bool progress = false;
      for (RadixNode* leaf : leaves) {
        if (freed >= want) break;
        for (int b : leaf->blocks) { unref(b); ++freed; ++evictions; }
        evictable_blocks -= (i64)leaf->blocks.size();
        RadixNode* parent = leaf->parent;
        parent->children.erase(edge_key(leaf->tokens.data()));
        delete leaf;
        progress = true;
      }
      if (!progress) break;
    }
    return freed;
  }

  void flush() {
    if (mode == 1) {
      hash_to_block.clear();
      std::fill(block_hashed.begin(), block_hashed.end(), 0);
      for (auto& v : block_tokens) v.clear();
    } else if (mode == 2) {
      // drop every unlocked subtree; locked paths stay until their sequences finish
      evict(pool.num_blocks);
    }
  }
};

// ------------------------------------------------------------------------------------------
enum SeqStatus { WAITING = 0, RUNNING = 1, FINISHED = 2 };

struct Seq {
  i64 id;
  std::vector<int> tokens;        // prompt + generated
  std::vector<float> logprobs;    // one per generated token
  int n_prompt = 0;
  int n_computed = 0;             // tokens whose KV is in the cache
  int n_cached = 0;               // prefix tokens served from the cache at the last admission
  std::vector<int> blocks;
  RadixNode* radix_node = nullptr;
  uint64_t chain = 0;             // hash chain over full blocks (hash mode)
  int n_hashed_blocks = 0;
  int status = WAITING;
  int max_new = 0;
  float temperature = 1.f;
  uint64_t seed = 0;
  std::vector<int> stop_ids;
  int eos = -1;
  int finish_reason = 0;          // 0 length, 1 stop
  int n_preempt = 0;
};

struct EngineCore {
  KVManager kv;
  int max_batch, max_tokens_per_batch, max_model_len;
  std::unordered_map<i64, std::unique_ptr<Seq>> seqs;
  std::deque<i64> waiting;
  std::vector<i64> running;
  i64 next_id = 0;
  // last schedule
  std::vector<i64> sched_prefill, sched_decode, sched_preempted;
  std::vector<i64> finished;

  EngineCore(int nb, int bs, int mode, int mb, int mt, int ml)
      : kv(nb, bs, mode), max_batch(mb), max_tokens_per_batch(mt), max_model_len(ml) {}

  Seq* get(i64 id) {
    auto it = seqs.find(id);
    return it == seqs.end() ? nullptr : it->second.get();
  }

  void release_blocks(Seq* s, bool publish) {
    const int bs = kv.pool.block_size;
    if (kv.mode == 2) {
      if (publish) {
        const int n_full = std::min((int)s->blocks.size(), s->n_computed / bs);
        if (n_full > 0) kv.insert_radix(s->tokens.data(), n_full, s->blocks.data());
      }
      if (s->radix_node) kv.lock_path(s->radix_node, -1);
      s->radix_node = nullptr;
    }
    for (int i = (int)s->blocks.size() - 1; i >= 0; --i) kv.unref(s->blocks[i]);
    s->blocks.clear();
    s->n_computed = 0;
    s->n_hashed_blocks = 0;
    s->chain = 0;
  }

  // Blocks a waiting sequence needs beyond what the prefix cache can serve is not known until
  // admission; the scheduler budgets with the conservative full count like the reference.
  bool admit(Seq* s) {
    const int bs = kv.pool.block_size;
    const int n = (int)s->tokens.size();
    const int need = (n + bs - 1) / bs;
    const int n_full_lookup = (n - 1) / bs;  // always recompute at least the last token
    std::vector<int> got;
    int matched = 0;
    if (kv.mode == 1) {
      matched = kv.match_hash(s->tokens.data(), n_full_lookup, got, s->chain);
      s->n_hashed_blocks = matched;
    } else if (kv.mode == 2) {
      kv.match_radix(s->tokens.data(), n_full_lookup, got);
      matched = (int)got.size();
      for (int b : got) {
        if (kv.pool.ref[b] == 0) kv.pool.unlink(b);  // not expected: the tree holds a ref
        ++kv.pool.ref[b];
      }
    }
    if (need - matched > kv.num_free()) {
      // roll back
      for (int i = matched - 1; i >= 0; --i) kv.unref(got[i]);
      s->chain = 0; s->n_hashed_blocks = 0;
      return false;
    }
    s->blocks = got;
    for (int i = matched; i < need; ++i) {
      int b = kv.take_block();
      if (b < 0) {  // cannot happen after the check above, but never leak
        release_blocks(s, false);
        return false;
      }
      s->blocks.push_back(b);
    }
    s->n_cached = matched * bs;
    s->n_computed = matched * bs;
    kv.hit_tokens += matched * bs;
    kv.miss_tokens += n - matched * bs;
    if (kv.mode == 1) {
      // publish the hashes of the full blocks this prefill is about to compute
      const int n_full = n / bs;
      for (int i = s->n_hashed_blocks; i < n_full; ++i) {
        uint64_t h;
        kv.register_hash(s->blocks[i], s->tokens.data() + i * bs, s->chain, h);
        s->chain = h;
      }
      s->n_hashed_blocks = std::max(s->n_hashed_blocks, n_full);
    } else if (kv.mode == 2) {
      // Publish the prompt's full blocks right away so sequences admitted later in this same
      // step already share them (their KV is written by this step's prefill before any
      // attention kernel reads it), then pin the path down to the deepest node.
      const int n_full = n / bs;
      if (n_full > 0) kv.insert_radix(s->tokens.data(), n_full, s->blocks.data());
      std::vector<int> tmp;
      RadixNode* deep = kv.match_radix(s->tokens.data(), n_full, tmp);
      kv.lock_path(deep, +1);
      s->radix_node = deep;
    }
    return true;
  }

  void preempt(Seq* s) {
    release_blocks(s, false);
    s->status = WAITING;
    ++s->n_preempt;
    waiting.push_front(s->id);
  }

  // One scheduling decision. Decode-first, then admit waiting sequences.
  void schedule() {
    sched_prefill.clear(); sched_decode.clear(); sched_preempted.clear();
    const int bs = kv.pool.block_size;
    int batch_tokens = 0;
    // 1. running sequences decode; each may need one new block for its next token
    std::vector<i64> keep;
    for (size_t i = 0; i < running.size(); ++i) {
      Seq* s = get(running[i]);
      if ((int)keep.size() >= max_batch) { sched_preempted.push_back(s->id); continue; }
      keep.push_back(s->id);
    }
    // ensure block capacity for the token being appended this step; preempt from the back
    for (size_t i = 0; i < keep.size(); ++i) {
      Seq* s = get(keep[i]);
      if (s == nullptr || s->status != RUNNING) continue;
      const int n = (int)s->tokens.size();           // the last token's KV is written this step
      const int need = (n + bs - 1) / bs;
      bool ok = true;
      while ((int)s->blocks.size() < need) {
        int b = kv.take_block();
        while (b < 0) {
          // out of blocks: preempt the youngest running sequence other than s
          Seq* victim = nullptr;
          for (int j = (int)keep.size() - 1; j > (int)i; --j) {
            Seq* c = get(keep[j]);
            if (c && c->status == RUNNING) { victim = c; break; }
          }
          if (victim == nullptr) break;
          sched_preempted.push_back(victim->id);
          preempt(victim);
          b = kv.take_block();
        }
        if (b < 0) { ok = false; break; }
        s->blocks.push_back(b);
      }
      if (!ok) { sched_preempted.push_back(s->id); preempt(s); continue; }
      sched_decode.push_back(s->id);
      batch_tokens += 1;
    }
    for (i64 id : sched_preempted) {
      Seq* s = get(id);
      if (s && s->status == RUNNING) preempt(s);
    }
    running.erase(std::remove_if(running.begin(), running.end(), [&](i64 id) { Seq* s = get(id); return !s || s->status != RUNNING; }),
                  running.end());
    // 2. admit waiting sequences
    while (!waiting.empty()) {
      Seq* s = get(waiting.front());
      if (s == nullptr) { waiting.pop_front(); continue; }
      if ((int)(sched_prefill.size() + sched_decode.size()) >= max_batch) break;
      const int n = (int)s->tokens.size();
      if (batch_tokens + n > max_tokens_per_batch && !(sched_prefill.empty() && sched_decode.empty())) break;
      // sequences preempted in this very step wait for the next one
      if (std::find(sched_preempted.begin(), sched_preempted.end(), s->id) != sched_preempted.end()) break;
      if (!admit(s)) break;
      waiting.pop_front();
      s->status = RUNNING;
      running.push_back(s->id);
      sched_prefill.push_back(s->id);
      batch_tokens += n - s->n_computed;
    }
  }

  void finish(Seq* s, int reason) {
    s->status = FINISHED;
    s->finish_reason = reason;
    release_blocks(s, true);
    finished.push_back(s->id);
  }
};

}  // namespace

extern "C" {

void* rbe_create(int num_blocks, int block_size, int cache_mode, int max_batch, int max_tokens_per_batch,
                 int max_model_len) {
  if (num_blocks <= 0 || block_size <= 0 || max_batch <= 0) return nullptr;
  return new EngineCore(num_blocks, block_size, cache_mode, max_batch, max_tokens_per_batch, max_model_len);
}
void rbe_destroy(void* h) { delete static_cast<EngineCore*>(h); }

i64 rbe_add_request(void* h, const int* tokens, int n, int max_new, float temperature, unsigned long long seed,
                    const int* stop_ids, int n_stop, int eos) {
  auto* e = static_cast<EngineCore*>(h);
  if (n <= 0 || n + max_new > e->max_model_len) return -1;
  auto s = std::make_unique<Seq>();
  s->id = e->next_id++;
  s->tokens.assign(tokens, tokens + n);
  s->n_prompt = n;
  s->max_new = max_new;
  s->temperature = temperature;
  s->seed = seed;
  if (n_stop > 0) s->stop_ids.assign(stop_ids, stop_ids + n_stop);
  s->eos = eos;
  i64 id = s->id;
  e->seqs[id] = std::move(s);
  e->waiting.push_back(id);
  return id;
}

int rbe_num_waiting(void* h) { return (int)static_cast<EngineCore*>(h)->waiting.size(); }
int rbe_num_running(void* h) { return (int)static_cast<EngineCore*>(h)->running.size(); }
int rbe_num_free_blocks(void* h) { return static_cast<EngineCore*>(h)->kv.num_free(); }

// Runs the scheduler. counts = {n_prefill, n_decode, n_preempted, new_tokens, max_new_len, max_blocks}
int rbe_schedule(void* h, int* counts) {
  auto* e = static_cast<EngineCore*>(h);
  e->schedule();
  int new_tokens = 0, max_new = 0, max_blocks = 0;
  for (i64 id : e->sched_prefill) {
    Seq* s = e->get(id);
    int n = (int)s->tokens.size() - s->n_computed;
    new_tokens += n;
    max_new = std::max(max_new, n);
    max_blocks = std::max(max_blocks, (int)s->blocks.size());
  }
  for (i64 id : e->sched_decode) {
    Seq* s = e->get(id);
    new_tokens += 1;
    max_new = std::max(max_new, 1);
    max_blocks = std::max(max_blocks, (int)s->blocks.size());
  }
  counts[0] = (int)e->sched_prefill.size();
  counts[1] = (int)e->sched_decode.size();
  counts[2] = (int)e->sched_preempted.size();
  counts[3] = new_tokens;
  counts[4] = max_new;
  counts[5] = max_blocks;
  return counts[0] + counts[1];
}

int rbe_get_scheduled(void* h, i64* prefill, i64* decode, i64* preempted) {
  auto* e = static_cast<EngineCore*>(h);
  if (prefill) std::copy(e->sched_prefill.begin(), e->sched_prefill.end(), prefill);
  if (decode) std::copy(e->sched_decode.begin(), e->sched_decode.end(), decode);
  if (preempted) std::copy(e->sched_preempted.begin(), e->sched_preempted.end(), preempted);
  return 0;
}

// Builds one packed batch from the last schedule: which = 1 the decode sequences (one new
// token each), which = 2 the admitted prefill sequences (all tokens not yet in the cache).
// block_tables is [rows, bt_stride]; rows beyond the batch are left untouched.
// Returns the number of packed tokens, or -1 if a buffer is too small.
int rbe_build_batch(void* h, int which, int* tokens, int* positions, int* slots, int* cu_q, int* seq_lens,
                    int* block_tables, int bt_stride, float* temps, unsigned long long* seeds, int* sample_rows,
                    int max_tokens, int max_rows) {
  auto* e = static_cast<EngineCore*>(h);
  const int bs = e->kv.pool.block_size;
  const std::vector<i64>& order = which == 1 ? e->sched_decode : e->sched_prefill;
  if ((int)order.size() > max_rows) return -1;
  int t = 0, row = 0;
  cu_q[0] = 0;
  for (i64 id : order) {
    Seq* s = e->get(id);
    const int n = (int)s->tokens.size();
    const int start = which == 1 ? n - 1 : s->n_computed;
    if (t + (n - start) > max_tokens) return -1;
    if ((int)s->blocks.size() > bt_stride) return -1;
    for (int p = start; p < n; ++p, ++t) {
      tokens[t] = s->tokens[p];
      positions[t] = p;
      slots[t] = s->blocks[p / bs] * bs + (p % bs);
    }
    cu_q[row + 1] = t;
    seq_lens[row] = n;
    std::copy(s->blocks.begin(), s->blocks.end(), block_tables + (size_t)row * bt_stride);
    temps[row] = s->temperature;
    seeds[row] = s->seed + 0x9E3779B97F4A7C15ull * (unsigned long long)(n - s->n_prompt);
    sample_rows[row] = t - 1;
    ++row;
  }
  return t;
}

// Appends the sampled token of every row of the decode (which = 1) or prefill (which = 2)
// batch, publishes blocks that just filled up to the prefix index, and applies the stop
// rules. Returns the number of sequences that finished.
int rbe_commit(void* h, int which, const int* sampled, const float* logprobs, int n_rows) {
  auto* e = static_cast<EngineCore*>(h);
  const int bs = e->kv.pool.block_size;
  const std::vector<i64> order = which == 1 ? e->sched_decode : e->sched_prefill;
  if (n_rows != (int)order.size()) return -1;
  int n_fin = 0;
  for (int r = 0; r < n_rows; ++r) {
    Seq* s = e->get(order[r]);
    if (s == nullptr || s->status != RUNNING) continue;
    s->n_computed = (int)s->tokens.size();
    if (e->kv.mode == 1) {
      const int n_full = s->n_computed / bs;
      for (int i = s->n_hashed_blocks; i < n_full && i < (int)s->blocks.size(); ++i) {
        uint64_t hsh;
        e->kv.register_hash(s->blocks[i], s->tokens.data() + i * bs, s->chain, hsh);
        s->chain = hsh;
      }
      s->n_hashed_blocks = std::max(s->n_hashed_blocks, n_full);
    }
    const int tok = sampled[r];
    s->tokens.push_back(tok);
    s->logprobs.push_back(logprobs[r]);
    const int n_gen = (int)s->tokens.size() - s->n_prompt;
    bool stop = tok == s->eos;
    for (int sid : s->stop_ids) stop = stop || sid == tok;
    if (stop) { e->finish(s, 1); ++n_fin; }
    else if (n_gen >= s->max_new || (int)s->tokens.size() >= e->max_model_len) { e->finish(s, 0); ++n_fin; }
  }
  e->running.erase(std::remove_if(e->running.begin(), e->running.end(),
                                  [&](i64 id) { Seq* s = e->get(id); return !s || s->status != RUNNING; }),
                   e->running.end());
  return n_fin;
}

int rbe_num_finished(void* h) { return (int)static_cast<EngineCore*>(h)->finished.size(); }

// Pops one finished sequence. info = {n_prompt, n_total, finish_reason, n_cached, n_preempt}
i64 rbe_pop_finished(void* h, int* info) {
  auto* e = static_cast<EngineCore*>(h);
  if (e->finished.empty()) return -1;
  i64 id = e->finished.front();
  e->finished.erase(e->finished.begin());
  Seq* s = e->get(id);
  info[0] = s->n_prompt;
  info[1] = (int)s->tokens.size();
  info[2] = s->finish_reason;
  info[3] = s->n_cached;
  info[4] = s->n_preempt;
  return id;
}
int rbe_read_sequence(void* h, i64 id, int* tokens, float* logprobs, int release) {
  auto* e = static_cast<EngineCore*>(h);
  Seq* s = e->get(id);
  if (!s) return -1;
  std::copy(s->tokens.begin(), s->tokens.end(), tokens);
  std::copy(s->logprobs.begin(), s->logprobs.end(), logprobs);
  if (release) e->seqs.erase(id);
  return 0;
}
int rbe_abort(void* h, i64 id) {
  auto* e = static_cast<EngineCore*>(h);
  Seq* s = e->get(id);
  if (!s) return -1;
  if (s->status == RUNNING) e->release_blocks(s, false);
  e->waiting.erase(std::remove(e->waiting.begin(), e->waiting.end(), id), e->waiting.end());
  e->running.erase(std::remove(e->running.begin(), e->running.end(), id), e->running.end());
  e->seqs.erase(id);
  return 0;
}
void rbe_flush_cache(void* h) { static_cast<EngineCore*>(h)->kv.flush(); }

// stats = {hit_tokens, miss_tokens, evictions, free_blocks, evictable_blocks}
void rbe_stats(void* h, i64* stats) {
  auto* e = static_cast<EngineCore*>(h);
  stats[0] = e->kv.hit_tokens; stats[1] = e->kv.miss_tokens; stats[2] = e->kv.evictions;
  stats[3] = e->kv.pool.free_count; stats[4] = e->kv.evictable_blocks;
}

// Allocator invariants: every refcount >= 0, a block is on the free list iff refcount == 0,
// and free + referenced == total. Returns 0 when they hold.
int rbe_check_invariants(void* h) {
  auto* e = static_cast<EngineCore*>(h);
  const BlockPool& p = e->kv.pool;
  int free_n = 0, used = 0;
  for (int b = 0; b < p.num_blocks; ++b) {
    if (p.ref[b] < 0) return 1;
    if ((p.ref[b] == 0) != (p.in_free[b] != 0)) return 2;
    if (p.in_free[b]) ++free_n; else ++used;
  }
  if (free_n != p.free_count) return 3;
  if (free_n + used != p.num_blocks) return 4;
  return 0;
}

// ---- stateless twins used by the Python-level API and the parity tests --------------------
// Pure scheduling policy of the reference over plain arrays.
//   running_ids/running_n, waiting_ids/waiting_lens; outputs are id arrays; counts[3].
void rb_schedule_pure(const i64* running_ids, int n_running, const i64* waiting_ids, const int* waiting_lens,
                      int n_waiting, int num_free_blocks, int max_batch, int max_tokens, int block_size,
                      i64* prefill, i64* decode, i64* preempted, int* counts) {
  int np = 0, nd = 0, npre = 0, batch_tokens = 0, blocks = num_free_blocks;
  for (int i = 0; i < n_running; ++i) {
    if (nd >= max_batch) { preempted[npre++] = running_ids[i]; continue; }
    decode[nd++] = running_ids[i];
    batch_tokens += 1;
  }
  for (int i = 0; i < n_waiting; ++i) {
    if (np + nd >= max_batch) break;
    const int n = waiting_lens[i];
    if (batch_tokens + n > max_tokens) break;
    const int need = (n + block_size - 1) / block_size;
    if (need > blocks) break;
    prefill[np++] = waiting_ids[i];
    blocks -= need;
    batch_tokens += n;
  }
  counts[0] = np; counts[1] = nd; counts[2] = npre;
}

// Stand-alone KV manager for the PagedKVCache / RadixKVCache Python classes. It re-uses the
// engine core's sequence table and admission logic without the scheduler.
void* rbk_create(int num_blocks, int block_size, int mode) {
  return new EngineCore(num_blocks, block_size, mode, 1 << 30, 1 << 30, 1 << 30);
}
// Allocates blocks for a new sequence; returns the number of blocks (-1: exists, -2: no room).
int rbk_allocate(void* h, i64 seq_id, const int* tokens, int n, int* out_blocks, int max_out, int* cached) {
  auto* e = static_cast<EngineCore*>(h);
  if (e->get(seq_id) != nullptr) return -1;
  auto s = std::make_unique<Seq>();
  s->id = seq_id;
  s->tokens.assign(tokens, tokens + n);
  s->n_prompt = n;
  Seq* sp = s.get();
  if (!e->admit(sp)) return -2;
  if ((int)sp->blocks.size() > max_out) { e->release_blocks(sp, false); return -3; }
  sp->status = RUNNING;
  sp->n_computed = n;
  std::copy(sp->blocks.begin(), sp->blocks.end(), out_blocks);
  *cached = sp->n_cached;
  e->seqs[seq_id] = std::move(s);
  return (int)sp->blocks.size();
}
// Appends one token; returns the id of a newly allocated block, -1 if none was needed,
// -2 if the pool is exhausted, -3 for an unknown sequence.
int rbk_append_token(void* h, i64 seq_id, int token) {
  auto* e = static_cast<EngineCore*>(h);
  Seq* s = e->get(seq_id);
  if (!s) return -3;
  const int bs = e->kv.pool.block_size;
  int new_block = -1;
  if ((int)s->tokens.size() + 1 > (int)s->blocks.size() * bs) {
    int b = e->kv.take_block();
    if (b < 0) return -2;
    s->blocks.push_back(b);
    new_block = b;
  }
  s->tokens.push_back(token);
  s->n_computed = (int)s->tokens.size();
  if (e->kv.mode == 1) {
    const int n_full = s->n_computed / bs;
    for (int i = s->n_hashed_blocks; i < n_full; ++i) {
      uint64_t hsh;
      e->kv.register_hash(s->blocks[i], s->tokens.data() + i * bs, s->chain, hsh);
      s->chain = hsh;
    }
    s->n_hashed_blocks = std::max(s->n_hashed_blocks, n_full);
  }
  return new_block;
}
int rbk_deallocate(void* h, i64 seq_id, int publish) {
  auto* e = static_cast<EngineCore*>(h);
  Seq* s = e->get(seq_id);
  if (!s) return -1;
  e->release_blocks(s, publish != 0);
  e->seqs.erase(seq_id);
  return 0;
}
int rbk_get_blocks(void* h, i64 seq_id, int* out, int max_out) {
  auto* e = static_cast<EngineCore*>(h);
  Seq* s = e->get(seq_id);
  if (!s) return -1;
  const int n = std::min((int)s->blocks.size(), max_out);
  std::copy(s->blocks.begin(), s->blocks.begin() + n, out);
  return (int)s->blocks.size();
}
int rbk_cached_tokens(void* h, i64 seq_id) {
  auto* e = static_cast<EngineCore*>(h);
  Seq* s = e->get(seq_id);
  return s ? s->n_cached : -1;
}
int rbk_ref_count(void* h, int block) {
  auto* e = static_cast<EngineCore*>(h);
  if (block < 0 || block >= e->kv.pool.num_blocks) return -1;
  return e->kv.pool.ref[block];
}

}  // extern "C"
