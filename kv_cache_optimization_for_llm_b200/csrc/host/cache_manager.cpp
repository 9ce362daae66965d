#include "cache_manager.h"

#include <algorithm>
#include <sstream>
#include <stdexcept>

namespace kvb {

CacheManager::CacheManager(std::vector<GroupSpec> groups, std::vector<int> pages_per_group,
                           int num_slots)
    : groups_(std::move(groups)) {
  if (groups_.size() != pages_per_group.size())
    throw std::invalid_argument("CacheManager: one page count per group is required");
  if (num_slots < 1) throw std::invalid_argument("CacheManager: num_slots must be >= 1");
  for (size_t g = 0; g < groups_.size(); ++g) {
    if (groups_[g].page_size < 1 || groups_[g].window < 0 || pages_per_group[g] < 1)
      throw std::invalid_argument("CacheManager: bad geometry for group " + std::to_string(g));
    // Free list starts 0..N-1 and is popped from the back, as upstream's is
    // (paged_attention/src/engine.cu:216-217,376-382): a page given back is the
    // next one handed out, so reuse is immediate.
    std::vector<int> fl(pages_per_group[g]);
    for (int p = 0; p < pages_per_group[g]; ++p) fl[p] = p;
    free_.push_back(std::move(fl));
    owner_.emplace_back(pages_per_group[g], kFree);
  }
  slot_owner_.assign(num_slots, kFree);
  for (int s = num_slots - 1; s >= 0; --s) free_slots_.push_back(s);
}

const CacheManager::Req& CacheManager::req(int64_t id) const {
  auto it = reqs_.find(id);
  if (it == reqs_.end())
    throw std::out_of_range("CacheManager: unknown request " + std::to_string(id));
  return it->second;
}
CacheManager::Req& CacheManager::req(int64_t id) {
  return const_cast<Req&>(static_cast<const CacheManager*>(this)->req(id));
}

int CacheManager::admit(int64_t id) {
  if (id == kFree) throw std::invalid_argument("CacheManager: reserved request id");
  if (reqs_.count(id))
    throw std::invalid_argument("CacheManager: request " + std::to_string(id) + " is already live");
  if (free_slots_.empty()) return -1;
  Req r;
  r.slot = free_slots_.back();
  free_slots_.pop_back();
  slot_owner_[r.slot] = id;
  r.tables.resize(groups_.size());
  const int slot = r.slot;
  reqs_.emplace(id, std::move(r));
  return slot;
}

int CacheManager::slot_of(int64_t id) const { return req(id).slot; }
int CacheManager::computed(int64_t id) const { return req(id).computed; }

int CacheManager::first_needed_token(int g, int computed) const {
  const int w = groups_[g].window;
  if (w <= 0) return 0;
  // The next query sits at position >= computed and reads keys > position - w.
  return std::max(0, computed - w + 1);
}

std::vector<int> CacheManager::pages_needed(int64_t id, int new_len) const {
  const Req& r = req(id);
  std::vector<int> need(groups_.size(), 0);
  for (size_t g = 0; g < groups_.size(); ++g) {
    const int ps = groups_[g].page_size;
    const int first = first_needed_token((int)g, r.computed) / ps;
    const int last = (new_len + ps - 1) / ps;  // exclusive
    for (int lp = first; lp < last; ++lp)
      if (lp >= (int)r.tables[g].size() || r.tables[g][lp] < 0) ++need[g];
  }
  return need;
}

bool CacheManager::extend(int64_t id, int new_len) {
  Req& r = req(id);
  if (new_len < r.computed)
    throw std::invalid_argument("CacheManager: extend below the computed length");
  const std::vector<int> need = pages_needed(id, new_len);
  for (size_t g = 0; g < groups_.size(); ++g)
    if (need[g] > (int)free_[g].size()) return false;
  for (size_t g = 0; g < groups_.size(); ++g) {
    const int ps = groups_[g].page_size;
    const int first = first_needed_token((int)g, r.computed) / ps;
    const int last = (new_len + ps - 1) / ps;
    if ((int)r.tables[g].size() < last) r.tables[g].resize(last, -1);
    for (int lp = first; lp < last; ++lp) {
      if (r.tables[g][lp] >= 0) continue;
      const int page = free_[g].back();
      free_[g].pop_back();
      owner_[g][page] = id;
      r.tables[g][lp] = page;
      ++taken_total_;
    }
  }
  return true;
}

void CacheManager::give_back(int g, int page) {
  if (page < 0 || page >= (int)owner_[g].size() || owner_[g][page] == kFree)
    throw std::logic_error("CacheManager: page " + std::to_string(page) + " of group " +
                           std::to_string(g) + " is given back but not held");
  owner_[g][page] = kFree;
  free_[g].push_back(page);
}

void CacheManager::advance(int64_t id, int computed) {
  Req& r = req(id);
  if (computed < r.computed)
    throw std::invalid_argument("CacheManager: advance moves backwards");
  r.computed = computed;
  for (size_t g = 0; g < groups_.size(); ++g) {
    if (groups_[g].window <= 0) continue;
    const int keep_from = first_needed_token((int)g, computed) / groups_[g].page_size;
    const int upto = std::min<int>(keep_from, (int)r.tables[g].size());
    for (int lp = 0; lp < upto; ++lp) {
      if (r.tables[g][lp] < 0) continue;
      give_back((int)g, r.tables[g][lp]);
      r.tables[g][lp] = -1;
    }
  }
}

void CacheManager::drop_pages(int64_t id) {
  Req& r = req(id);
  for (size_t g = 0; g < groups_.size(); ++g) {
    // Back to front, so that the LIFO list hands the lowest logical page's
    // physical page out first again.
    for (int lp = (int)r.tables[g].size() - 1; lp >= 0; --lp)
      if (r.tables[g][lp] >= 0) give_back((int)g, r.tables[g][lp]);
    r.tables[g].clear();
  }
  r.computed = 0;
}

void CacheManager::release(int64_t id) {
  drop_pages(id);
  Req& r = req(id);
  slot_owner_[r.slot] = kFree;
  free_slots_.push_back(r.slot);
  reqs_.erase(id);
}

const std::vector<int>& CacheManager::block_table(int64_t id, int group) const {
  return req(id).tables.at(group);
}

std::string CacheManager::check() const {
  std::ostringstream err;
  for (size_t g = 0; g < groups_.size(); ++g) {
    const int n = (int)owner_[g].size();
    std::vector<int> seen_free(n, 0), seen_held(n, 0);
    for (int p : free_[g]) {
      if (p < 0 || p >= n) { err << "group " << g << ": free list holds bad page " << p << "; "; continue; }
      if (++seen_free[p] > 1) err << "group " << g << ": page " << p << " is free twice; ";
      if (owner_[g][p] != kFree) err << "group " << g << ": free page " << p << " has an owner; ";
    }
    for (const auto& kv : reqs_) {
      for (int p : kv.second.tables[g]) {
        if (p < 0) continue;
        if (p >= n) { err << "group " << g << ": request " << kv.first << " holds bad page " << p << "; "; continue; }
        if (++seen_held[p] > 1) err << "group " << g << ": page " << p << " is held twice; ";
        if (owner_[g][p] != kv.first) err << "group " << g << ": page " << p << " owner mismatch; ";
      }
    }
    for (int p = 0; p < n; ++p)
      if (seen_free[p] + seen_held[p] != 1)
        err << "group " << g << ": page " << p << " is " << (seen_free[p] + seen_held[p] ? "both free and held" : "lost") << "; ";
  }
  const int ns = (int)slot_owner_.size();
  std::vector<int> slot_seen(ns, 0);
  for (int s : free_slots_) {
    if (s < 0 || s >= ns) { err << "bad free slot " << s << "; "; continue; }
    if (++slot_seen[s] > 1) err << "slot " << s << " is free twice; ";
    if (slot_owner_[s] != kFree) err << "free slot " << s << " has an owner; ";
  }
  for (const auto& kv : reqs_) {
    const int s = kv.second.slot;
    if (s < 0 || s >= ns) { err << "request " << kv.first << " has bad slot; "; continue; }
    if (++slot_seen[s] > 1) err << "slot " << s << " is held twice; ";
    if (slot_owner_[s] != kv.first) err << "slot " << s << " owner mismatch; ";
  }
  for (int s = 0; s < ns; ++s)
    if (slot_seen[s] != 1) err << "slot " << s << " is lost; ";
  return err.str();
}

}  // namespace kvb
