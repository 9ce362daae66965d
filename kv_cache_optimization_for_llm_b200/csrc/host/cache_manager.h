// Paged cache bookkeeping: which physical pages and which state slot every live
// request holds.  It owns integers only; the device tensors that the pages and
// slots index are allocated by the Python side from the same geometry.
//
// Counterpart of the upstream paged build's KVCacheState / kvTakePage /
// kvDropPage / finishSequence / kvPageAccountingHolds
// (paged_attention/src/engine.cuh:135-178, paged_attention/src/engine.cu:376-475),
// redesigned: one page id covers every layer of its group, each request owns a
// plain list of pages per group, and layers with different needs (all keys, or a
// sliding window of them) live in groups with pools of their own.
#pragma once

#include <cstdint>
#include <string>
#include <unordered_map>
#include <vector>

namespace kvb {

struct GroupSpec {
  int page_size = 16;  // tokens per page
  int window = 0;      // 0: every key is kept; W>0: only the newest W keys are read
};

class CacheManager {
 public:
  CacheManager(std::vector<GroupSpec> groups, std::vector<int> pages_per_group, int num_slots);

  // Registers a request and gives it a state slot.  Returns the slot, or -1 when
  // no slot is free (nothing changes then).  Throws if the id is already live.
  int admit(int64_t id);
  bool has(int64_t id) const { return reqs_.count(id) != 0; }
  int slot_of(int64_t id) const;
  int computed(int64_t id) const;  // tokens whose keys are in the cache

  // Pages that extend(id, new_len) would have to take, per group.
  std::vector<int> pages_needed(int64_t id, int new_len) const;
  // Makes pages cover every token that a step computing [computed, new_len) reads
  // or writes, in every group, or changes nothing and returns false.
  bool extend(int64_t id, int new_len);
  // Records that tokens [0, computed) are now in the cache and gives back the
  // pages that a window has passed for good.
  void advance(int64_t id, int computed);
  // Gives back every page and the slot.
  void release(int64_t id);
  // Gives back the pages, keeps the slot and the registration (recompute from 0).
  void drop_pages(int64_t id);

  // Logical page number -> physical page, -1 where no page is held.
  const std::vector<int>& block_table(int64_t id, int group) const;

  int num_groups() const { return (int)groups_.size(); }
  const GroupSpec& group(int g) const { return groups_.at(g); }
  int num_pages(int g) const { return (int)owner_.at(g).size(); }
  int free_pages(int g) const { return (int)free_.at(g).size(); }
  int num_slots() const { return (int)slot_owner_.size(); }
  int free_slots() const { return (int)free_slots_.size(); }
  int live_requests() const { return (int)reqs_.size(); }
  int64_t pages_taken_total() const { return taken_total_; }

  // Empty when the accounting holds: every page is either free once or held once
  // by exactly the request its owner entry names; same for slots.
  std::string check() const;

 private:
  struct Req {
    int slot = -1;
    int computed = 0;
    std::vector<std::vector<int>> tables;  // [group][logical page]
  };
  static constexpr int64_t kFree = INT64_MIN;

  int first_needed_token(int g, int computed) const;
  void give_back(int g, int page);
  const Req& req(int64_t id) const;
  Req& req(int64_t id);

  std::vector<GroupSpec> groups_;
  std::vector<std::vector<int>> free_;       // LIFO free lists
  std::vector<std::vector<int64_t>> owner_;  // [group][page] -> request id or kFree
  std::vector<int> free_slots_;
  std::vector<int64_t> slot_owner_;
  std::unordered_map<int64_t, Req> reqs_;
  int64_t taken_total_ = 0;
};

}  // namespace kvb
