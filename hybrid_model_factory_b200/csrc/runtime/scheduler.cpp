// Serving runtime core (host only): paged KV block manager with hash-chained prefix caching, fixed-size
// recurrent-state slots for SSM layers (with "align"-mode snapshots at block boundaries so that a cached
// prefix of a hybrid model can be resumed), and a continuous-batching scheduler with chunked prefill that
// places decodes first in every batch.  Exposed as a C API and bound from Python with ctypes
// (serving/scheduler.py).  Behavioural model: what the reference project obtains from vLLM's scheduler,
// hybrid KV-cache manager and `--mamba-cache-mode align` (docs/Inference.md:153-165, 233-245).
#include <stdint.h>
#include <string.h>

#include <algorithm>
#include <deque>
#include <mutex>
#include <unordered_map>
#include <vector>

#define HMF_API extern "C" __attribute__((visibility("default")))

namespace {

struct Request {
  int64_t id;
  std::vector<int32_t> tokens;   // prompt + generated
  int prompt_len = 0;
  int max_new_tokens = 0;
  int computed = 0;              // tokens whose KV / state are in the cache
  int slot = -1;                 // recurrent-state slot
  std::vector<int32_t> blocks;   // KV block table
  bool finished = false;
  bool running = false;
  int cached_prefix = 0;         // tokens served from the prefix cache at admission
  int snapshot_slot = -1;        // state snapshot to restore from (align mode) or -1
};

struct Block {
  int ref = 0;
  uint64_t hash = 0;
  bool hashed = false;
  uint64_t last_use = 0;
};

struct Snapshot {
  int slot;
  uint64_t last_use;
};

class Scheduler {
 public:
  Scheduler(int num_blocks, int block_size, int num_slots, int max_seqs, int max_tokens, int prefix_cache,
            int num_snapshot_slots)
      : block_size_(block_size), max_seqs_(max_seqs), max_tokens_(max_tokens), prefix_cache_(prefix_cache != 0),
        blocks_(num_blocks) {
    for (int i = num_blocks - 1; i >= 0; --i) free_blocks_.push_back(i);
    for (int i = num_slots - 1; i >= 0; --i) free_slots_.push_back(i);
    // snapshot slots live after the request slots in the same state tensors
    for (int i = num_snapshot_slots - 1; i >= 0; --i) free_snap_slots_.push_back(num_slots + i);
  }

  int add(int64_t id, const int32_t* prompt, int n, int max_new) {
    std::lock_guard<std::mutex> g(mu_);
    if (reqs_.count(id)) return -1;
    Request r;
    r.id = id;
    r.tokens.assign(prompt, prompt + n);
    r.prompt_len = n;
    r.max_new_tokens = max_new;
    reqs_[id] = std::move(r);
    waiting_.push_back(id);
    return 0;
  }

  // One scheduling step.  Output rows: (req_id, num_tokens, start_pos, slot, restore_from_slot).
  int step(int64_t* ids, int32_t* ntok, int32_t* start, int32_t* slots, int32_t* restore, int max_out) {
    std::lock_guard<std::mutex> g(mu_);
    ++clock_;
    int n_out = 0, budget = max_tokens_;
    // 1. decodes first: one token each
    for (int64_t id : running_) {
      Request& r = reqs_[id];
      if (r.finished || r.computed < r.prompt_len) continue;
      if (n_out >= max_out || budget <= 0) break;
      if (!ensure_blocks(r, r.computed + 1)) { preempt_later_.push_back(id); continue; }
      ids[n_out] = id; ntok[n_out] = 1; start[n_out] = r.computed; slots[n_out] = r.slot; restore[n_out] = -1;
      ++n_out; --budget;
    }
    // 2. running prefills continue (chunked)
    int prefill_used = 0;
    for (int64_t id : running_) {
      Request& r = reqs_[id];
      if (r.finished || r.computed >= r.prompt_len) continue;
      if (n_out >= max_out || budget <= 0) break;
      int chunk = std::min(budget, r.prompt_len - r.computed);
      chunk = align_chunk(r, chunk);
      if (chunk <= 0 || !ensure_blocks(r, r.computed + chunk)) continue;
      ids[n_out] = id; ntok[n_out] = chunk; start[n_out] = r.computed; slots[n_out] = r.slot; restore[n_out] = -1;
      ++n_out; budget -= chunk; prefill_used += chunk;
    }
    // 3. admit waiting requests
    const int prefill_budget = budget + prefill_used;
    while (!waiting_.empty() && (int)running_.size() < max_seqs_ && n_out < max_out && budget > 0) {
      int64_t id = waiting_.front();
      Request& r = reqs_[id];
      if (free_slots_.empty()) break;
      int hit = prefix_cache_ ? lookup_prefix(r) : 0;
      // whole-prompt policy: a prompt that would fit a step of its own is not split just to fill the rest of this one
      // (every scheduled piece is a separate forward pass of the engine, so fewer and larger pieces run faster)
      if (whole_prompts_ && budget < prefill_budget && r.prompt_len - hit > budget && r.prompt_len - hit <= prefill_budget)
        break;
      int chunk = std::min(budget, r.prompt_len - hit);
      r.computed = hit;
      chunk = align_chunk(r, chunk);
      if (chunk <= 0 || !ensure_blocks(r, hit + chunk)) {
        release_blocks(r);
        r.computed = 0;
        break;
      }
      waiting_.pop_front();
      r.slot = free_slots_.back();
      free_slots_.pop_back();
      r.running = true;
      r.cached_prefix = hit;
      running_.push_back(id);
      ids[n_out] = id; ntok[n_out] = chunk; start[n_out] = hit; slots[n_out] = r.slot; restore[n_out] = r.snapshot_slot;
      ++n_out; budget -= chunk;
    }
    preempt_later_.clear();
    return n_out;
  }

  // Called after the model ran the scheduled tokens of a request.
  void advance(int64_t id, int n) {
    std::lock_guard<std::mutex> g(mu_);
    auto it = reqs_.find(id);
    if (it == reqs_.end()) return;
    Request& r = it->second;
    r.computed += n;
    if (prefix_cache_) hash_full_blocks(r);
  }

  void append_token(int64_t id, int32_t tok) {
    std::lock_guard<std::mutex> g(mu_);
    auto it = reqs_.find(id);
    if (it == reqs_.end()) return;
    it->second.tokens.push_back(tok);
    if ((int)it->second.tokens.size() - it->second.prompt_len >= it->second.max_new_tokens) it->second.finished = true;
  }

  int finish(int64_t id) {
    std::lock_guard<std::mutex> g(mu_);
    auto it = reqs_.find(id);
    if (it == reqs_.end()) return -1;
    Request& r = it->second;
    release_blocks(r);
    if (r.slot >= 0) free_slots_.push_back(r.slot);
    running_.erase(std::remove(running_.begin(), running_.end(), id), running_.end());
    waiting_.erase(std::remove(waiting_.begin(), waiting_.end(), id), waiting_.end());
    reqs_.erase(it);
    return 0;
  }

  int block_table(int64_t id, int32_t* out, int max_n) {
    std::lock_guard<std::mutex> g(mu_);
    auto it = reqs_.find(id);
    if (it == reqs_.end()) return -1;
    int n = std::min<int>(max_n, it->second.blocks.size());
    memcpy(out, it->second.blocks.data(), n * sizeof(int32_t));
    return (int)it->second.blocks.size();
  }

  // align mode: the engine saved the recurrent state of request `id` at position `pos` (a block boundary)
  // into snapshot slot returned here (-1: no slot available).
  int register_snapshot(int64_t id, int pos) {
    std::lock_guard<std::mutex> g(mu_);
    auto it = reqs_.find(id);
    if (it == reqs_.end() || pos % block_size_ != 0 || pos <= 0) return -1;
    uint64_t h = chain_hash(it->second, pos / block_size_);
    auto s = snapshots_.find(h);
    if (s != snapshots_.end()) { s->second.last_use = clock_; return -2; }  // already stored
    int slot;
    if (!free_snap_slots_.empty()) {
      slot = free_snap_slots_.back();
      free_snap_slots_.pop_back();
    } else {
      if (snapshots_.empty()) return -1;
      auto victim = snapshots_.begin();
      for (auto i = snapshots_.begin(); i != snapshots_.end(); ++i)
        if (i->second.last_use < victim->second.last_use) victim = i;
      slot = victim->second.slot;
      snapshots_.erase(victim);
    }
    snapshots_[h] = Snapshot{slot, clock_};
    return slot;
  }

  void stats(int64_t* out) {
    std::lock_guard<std::mutex> g(mu_);
    out[0] = (int64_t)free_blocks_.size();
    out[1] = (int64_t)free_slots_.size();
    out[2] = (int64_t)running_.size();
    out[3] = (int64_t)waiting_.size();
    out[4] = prefix_hits_;
    out[5] = prefix_queries_;
    out[6] = (int64_t)snapshots_.size();
    out[7] = evictions_;
  }

  int is_finished(int64_t id) {
    std::lock_guard<std::mutex> g(mu_);
    auto it = reqs_.find(id);
    return it == reqs_.end() ? -1 : (it->second.finished ? 1 : 0);
  }

 private:
  static uint64_t mix(uint64_t h, uint64_t v) {
    h ^= v + 0x9e3779b97f4a7c15ull + (h << 6) + (h >> 2);
    return h * 0xff51afd7ed558ccdull;
  }
  uint64_t chain_hash(const Request& r, int n_blocks) const {
    uint64_t h = 0x12345678abcdefull;
    for (int b = 0; b < n_blocks; ++b)
      for (int i = 0; i < block_size_; ++i) h = mix(h, (uint64_t)(uint32_t)r.tokens[b * block_size_ + i]);
    return h;
  }
  // Chunk boundaries of a prefill end on block boundaries (except at the end of the prompt), so that state
  // snapshots taken at the end of a chunk are block aligned.
  int align_chunk(const Request& r, int chunk) const {
    if (r.computed + chunk >= r.prompt_len) return chunk;
    int end = (r.computed + chunk) / block_size_ * block_size_;
    return end - r.computed;
  }
  int alloc_block() {
    if (free_blocks_.empty()) {
      // evict the least recently used cached block that nobody references
      int victim = -1;
      for (auto& kv : cached_) {
        Block& b = blocks_[kv.second];
        if (b.ref == 0 && (victim < 0 || b.last_use < blocks_[victim].last_use)) victim = kv.second;
      }
      if (victim < 0) return -1;
      cached_.erase(blocks_[victim].hash);
      blocks_[victim].hashed = false;
      ++evictions_;
      return victim;
    }
    int b = free_blocks_.back();
    free_blocks_.pop_back();
    return b;
  }
  bool ensure_blocks(Request& r, int n_tokens) {
    int need = (n_tokens + block_size_ - 1) / block_size_;
    while ((int)r.blocks.size() < need) {
      int b = alloc_block();
      if (b < 0) return false;
      blocks_[b].ref = 1;
      blocks_[b].hashed = false;
      blocks_[b].last_use = clock_;
      r.blocks.push_back(b);
    }
    return true;
  }
  void release_blocks(Request& r) {
    for (int b : r.blocks) {
      Block& blk = blocks_[b];
      if (--blk.ref <= 0) {
        blk.ref = 0;
        blk.last_use = clock_;
        if (!blk.hashed) free_blocks_.push_back(b);  // hashed blocks stay as evictable cache entries
      }
    }
    r.blocks.clear();
  }
  // Longest cached prefix of full blocks; for hybrid models the hit is cut back to the longest prefix that
  // also has a recurrent-state snapshot (or kept as is when the model has no recurrent state: slot count 0).
  int lookup_prefix(Request& r) {
    ++prefix_queries_;
    int max_blocks = (r.prompt_len - 1) / block_size_;  // keep at least one token to compute
    uint64_t h = 0x12345678abcdefull;
    std::vector<int> hit_blocks;
    int best_snapshot_blocks = 0, best_snapshot_slot = -1;
    for (int b = 0; b < max_blocks; ++b) {
      for (int i = 0; i < block_size_; ++i) h = mix(h, (uint64_t)(uint32_t)r.tokens[b * block_size_ + i]);
      auto it = cached_.find(h);
      if (it == cached_.end()) break;
      hit_blocks.push_back(it->second);
      auto s = snapshots_.find(h);
      if (s != snapshots_.end()) { best_snapshot_blocks = b + 1; best_snapshot_slot = s->second.slot; s->second.last_use = clock_; }
    }
    int use_blocks = require_snapshot_ ? best_snapshot_blocks : (int)hit_blocks.size();
    for (int b = 0; b < use_blocks; ++b) {
      Block& blk = blocks_[hit_blocks[b]];
      if (blk.ref == 0) {
        // leaving the evictable set
      }
      ++blk.ref;
      blk.last_use = clock_;
      r.blocks.push_back(hit_blocks[b]);
    }
    r.snapshot_slot = require_snapshot_ && use_blocks > 0 ? best_snapshot_slot : -1;
    if (use_blocks > 0) ++prefix_hits_;
    return use_blocks * block_size_;
  }
  void hash_full_blocks(Request& r) {
    int full = std::min<int>(r.computed, (int)r.tokens.size()) / block_size_;
    uint64_t h = 0x12345678abcdefull;
    for (int b = 0; b < full && b < (int)r.blocks.size(); ++b) {
      for (int i = 0; i < block_size_; ++i) h = mix(h, (uint64_t)(uint32_t)r.tokens[b * block_size_ + i]);
      Block& blk = blocks_[r.blocks[b]];
      if (!blk.hashed && !cached_.count(h)) {
        blk.hashed = true;
        blk.hash = h;
        cached_[h] = r.blocks[b];
      }
    }
  }

 public:
  bool require_snapshot_ = false;
  bool whole_prompts_ = false;

 private:
  int block_size_, max_seqs_, max_tokens_;
  bool prefix_cache_;
  std::vector<Block> blocks_;
  std::vector<int> free_blocks_, free_slots_, free_snap_slots_;
  std::unordered_map<int64_t, Request> reqs_;
  std::deque<int64_t> waiting_;
  std::vector<int64_t> running_, preempt_later_;
  std::unordered_map<uint64_t, int> cached_;
  std::unordered_map<uint64_t, Snapshot> snapshots_;
  uint64_t clock_ = 0;
  int64_t prefix_hits_ = 0, prefix_queries_ = 0, evictions_ = 0;
  std::mutex mu_;
};

}  // namespace

HMF_API void* hmf_sched_create(int num_blocks, int block_size, int num_slots, int max_seqs, int max_tokens,
                               int prefix_cache, int num_snapshot_slots, int require_snapshot) {
  auto* s = new Scheduler(num_blocks, block_size, num_slots, max_seqs, max_tokens, prefix_cache, num_snapshot_slots);
  s->require_snapshot_ = require_snapshot != 0;
  return s;
}
HMF_API void hmf_sched_set_whole_prompts(void* s, int on) { static_cast<Scheduler*>(s)->whole_prompts_ = on != 0; }
HMF_API void hmf_sched_destroy(void* s) { delete static_cast<Scheduler*>(s); }
HMF_API int hmf_sched_add(void* s, int64_t id, const int32_t* prompt, int n, int max_new) {
  return static_cast<Scheduler*>(s)->add(id, prompt, n, max_new);
}
HMF_API int hmf_sched_step(void* s, int64_t* ids, int32_t* ntok, int32_t* start, int32_t* slots, int32_t* restore,
                           int max_out) {
  return static_cast<Scheduler*>(s)->step(ids, ntok, start, slots, restore, max_out);
}
HMF_API void hmf_sched_advance(void* s, int64_t id, int n) { static_cast<Scheduler*>(s)->advance(id, n); }
HMF_API void hmf_sched_append_token(void* s, int64_t id, int32_t tok) {
  static_cast<Scheduler*>(s)->append_token(id, tok);
}
HMF_API int hmf_sched_finish(void* s, int64_t id) { return static_cast<Scheduler*>(s)->finish(id); }
HMF_API int hmf_sched_block_table(void* s, int64_t id, int32_t* out, int max_n) {
  return static_cast<Scheduler*>(s)->block_table(id, out, max_n);
}
HMF_API int hmf_sched_register_snapshot(void* s, int64_t id, int pos) {
  return static_cast<Scheduler*>(s)->register_snapshot(id, pos);
}
HMF_API void hmf_sched_stats(void* s, int64_t* out) { static_cast<Scheduler*>(s)->stats(out); }
HMF_API int hmf_sched_is_finished(void* s, int64_t id) { return static_cast<Scheduler*>(s)->is_finished(id); }
