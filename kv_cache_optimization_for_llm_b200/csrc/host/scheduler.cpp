#include "scheduler.h"

#include <algorithm>
#include <stdexcept>

namespace kvb {

const char* finish_reason_name(FinishReason r) {
  switch (r) {
    case FinishReason::None: return "none";
    case FinishReason::Stop: return "stop";
    case FinishReason::Length: return "length";
    case FinishReason::ModelLen: return "sequence_too_long";
    case FinishReason::CacheExhausted: return "kv_cache_exhausted";
    case FinishReason::Aborted: return "aborted";
  }
  return "?";
}

Scheduler::Scheduler(CacheManager* cache, SchedulerConfig cfg) : cache_(cache), cfg_(cfg) {
  if (!cache_) throw std::invalid_argument("Scheduler: a cache manager is required");
  if (cfg_.max_num_seqs < 1 || cfg_.max_num_batched_tokens < 1 || cfg_.max_model_len < 2 ||
      cfg_.max_prefill_chunk < 0 || cfg_.max_portions_per_step < 0)
    throw std::invalid_argument("Scheduler: limits must be positive");
}

void Scheduler::add(int64_t id, std::vector<int> prompt, int max_tokens) {
  if (prompt.empty()) throw std::invalid_argument("Scheduler: request with an empty prompt");
  if (max_tokens < 1) throw std::invalid_argument("Scheduler: max_tokens must be >= 1");
  if (reqs_.count(id) || done_.count(id))
    throw std::invalid_argument("Scheduler: request id " + std::to_string(id) + " is in use");
  if ((int)prompt.size() >= cfg_.max_model_len)
    throw std::invalid_argument("Scheduler: a prompt of " + std::to_string(prompt.size()) +
                                " tokens leaves no room under max_model_len " +
                                std::to_string(cfg_.max_model_len));
  for (int g = 0; g < cache_->num_groups(); ++g) {
    const GroupSpec& gs = cache_->group(g);
    // A group that keeps every key must hold the whole prompt and one more token;
    // a windowed group at most the window plus one step's portion, which the
    // scheduler can shrink, so only the full groups decide.
    if (gs.window > 0) continue;
    const int need = ((int)prompt.size() + 1 + gs.page_size - 1) / gs.page_size;
    if (need > cache_->num_pages(g))
      throw std::invalid_argument("Scheduler: the prompt needs " + std::to_string(need) +
                                  " pages, the pool has " + std::to_string(cache_->num_pages(g)));
  }
  Req r;
  r.id = id;
  r.arrival = arrivals_++;
  r.prompt_len = (int)prompt.size();
  r.tokens = std::move(prompt);
  r.max_tokens = max_tokens;
  reqs_.emplace(id, std::move(r));
  waiting_.push_back(id);
}

const Scheduler::Req& Scheduler::any(int64_t id) const {
  auto it = reqs_.find(id);
  if (it != reqs_.end()) return it->second;
  it = done_.find(id);
  if (it != done_.end()) return it->second;
  throw std::out_of_range("Scheduler: unknown request " + std::to_string(id));
}

int Scheduler::portion(const Req& r, int budget) const {
  int n = std::min<int>((int)r.tokens.size() - r.computed, budget);
  if (cfg_.max_prefill_chunk > 0 && n > 1) n = std::min(n, cfg_.max_prefill_chunk);
  return n;
}

bool Scheduler::room_for_all_of(const Req& r) const {
  // Beside running requests a request is admitted only when the groups that keep every key have
  // free pages for all the tokens it has by now (its prompt, and what it produced before it was
  // dropped) and one more, plus a page of growth for each running request.  Admitting on the first
  // portion alone lets a long request in, reads part of it, and drops it again as soon as the
  // others grow: the same tokens are then computed over and over (upstream admits a prompt only
  // when all its pages are free, paged_attention/src/engine.cu:294-370).
  for (int g = 0; g < cache_->num_groups(); ++g) {
    const GroupSpec& gs = cache_->group(g);
    if (gs.window > 0) continue;
    const int need = ((int)r.tokens.size() + 1 + gs.page_size - 1) / gs.page_size;
    if (need + (int)running_.size() > cache_->free_pages(g)) return false;
  }
  return true;
}

int Scheduler::shrink_to_fit(const Req& r, int want) {
  // A portion needs pages for all its tokens at once, in a windowed group too, where the pages
  // that the window passes come back only after the step.  A request that nobody can make room
  // for tries smaller portions, halving down to one token, before it is given up: in a windowed
  // group the smaller portion is what lets a long prompt through a small pool.
  bool windowed = false;
  for (int g = 0; g < cache_->num_groups(); ++g) windowed = windowed || cache_->group(g).window > 0;
  if (!windowed) return 0;
  while (want > 1) {
    want = (want + 1) / 2;
    if (cache_->extend(r.id, r.computed + want)) return want;
  }
  return 0;
}

void Scheduler::finish(Req* r, FinishReason why) {
  const int64_t id = r->id;
  if (cache_->has(id)) cache_->release(id);
  running_.erase(std::remove(running_.begin(), running_.end(), id), running_.end());
  waiting_.erase(std::remove(waiting_.begin(), waiting_.end(), id), waiting_.end());
  if (r->pending) {   // ended before its newest tokens' values arrived: they are dropped
    r->tokens.resize(r->tokens.size() - r->pending);
    r->pending = 0;
    r->closing = false;
  }
  Req moved = std::move(*r);
  moved.reason = why;
  reqs_.erase(id);
  done_.emplace(id, std::move(moved));
  ++stats_.finished;
}

void Scheduler::preempt(size_t running_index, Plan* plan) {
  const int64_t id = running_[running_index];
  Req& r = reqs_.at(id);
  // Everything it holds goes back; its tokens (prompt and output so far) stay, and
  // are recomputed as an ordinary prompt when it is admitted again.  It arrived
  // before anything that still waits, so it goes to the front
  // (paged_attention/src/engine.cu:675-731).
  stats_.recomputed_tokens += r.computed;
  cache_->release(id);
  r.computed = 0;
  ++r.preemptions;
  ++stats_.preemptions;
  running_.erase(running_.begin() + running_index);
  waiting_.push_front(id);
  plan->preempted.push_back(id);
}

Plan Scheduler::schedule() {
  Plan plan;
  int budget = cfg_.max_num_batched_tokens;
  bool preempted_now = false;
  int portions = 0;   // runs of more than one token in this step
  auto no_more_portions = [&](int want) {
    return want > 1 && cfg_.max_portions_per_step > 0 && portions >= cfg_.max_portions_per_step;
  };

  // Running requests first, oldest first: one decode token each, or the next
  // portion of a prompt that is still being read.
  size_t i = 0;
  while (i < running_.size()) {
    Req& r = reqs_.at(running_[i]);
    int want = r.closing ? 0 : portion(r, budget);
    if (want <= 0) { ++i; continue; }  // budget spent (or only waiting for its last token): not in this step
    if (no_more_portions(want)) { ++i; continue; }   // its next portion waits for a step with room for a portion
    bool scheduled = true;
    while (!cache_->extend(r.id, r.computed + want)) {
      // Pages ran out.  The latest arrival among the running gives way, this
      // request itself if it is the latest.
      const size_t victim = running_.size() - 1;
      if (victim == i && running_.size() == 1) {
        const int smaller = shrink_to_fit(r, want);
        if (smaller > 0) { want = smaller; break; }   // its pages are in place
        // Alone and still too large for the pool: it can never finish.
        plan.finished.push_back(r.id);
        finish(&r, FinishReason::CacheExhausted);
        scheduled = false;
        break;
      }
      preempted_now = true;
      const bool self = (victim == i);
      preempt(victim, &plan);
      if (self) { scheduled = false; break; }
    }
    if (!scheduled) continue;  // running_[i] is gone or i is past the end
    PlanEntry e;
    e.id = r.id;
    e.start = r.computed;
    e.tokens.assign(r.tokens.begin() + r.computed, r.tokens.begin() + r.computed + want);
    e.sample = (r.computed + want == (int)r.tokens.size());
    plan.entries.push_back(std::move(e));
    plan.num_tokens += want;
    budget -= want;
    if (want > 1) ++portions;
    ++i;
  }

  // Then the queue, in order, while seats, budget and pages last.  Nothing new is
  // admitted in a step that had to preempt.
  while (!preempted_now && !waiting_.empty() && (int)running_.size() < cfg_.max_num_seqs &&
         budget > 0) {
    Req& r = reqs_.at(waiting_.front());
    if (r.pending) break;                // its newest token is not known yet: next step
    if (!running_.empty() && !room_for_all_of(r)) break;   // it would only be dropped again
    if (no_more_portions(portion(r, budget))) break;
    if (cache_->admit(r.id) < 0) break;  // no state slot free
    int want = portion(r, budget);
    if (!cache_->extend(r.id, want)) {
      const int smaller = running_.empty() ? shrink_to_fit(r, want) : 0;
      if (smaller > 0) {
        want = smaller;
      } else {
        cache_->release(r.id);
        if (running_.empty()) {
          plan.finished.push_back(r.id);
          finish(&r, FinishReason::CacheExhausted);
          continue;
        }
        break;
      }
    }
    waiting_.pop_front();
    running_.push_back(r.id);
    PlanEntry e;
    e.id = r.id;
    e.start = 0;
    e.tokens.assign(r.tokens.begin(), r.tokens.begin() + want);
    e.sample = (want == (int)r.tokens.size());
    plan.entries.push_back(std::move(e));
    plan.num_tokens += want;
    budget -= want;
    if (want > 1) ++portions;
  }
  return plan;
}

void Scheduler::commit(const Plan& plan) {
  for (const PlanEntry& e : plan.entries) {
    Req& r = reqs_.at(e.id);
    r.computed = e.start + (int)e.tokens.size();
    cache_->advance(e.id, r.computed);
  }
  ++stats_.steps;
  stats_.scheduled_tokens += plan.num_tokens;
}

FinishReason Scheduler::append_token(int64_t id, int token, bool is_stop) {
  Req& r = reqs_.at(id);
  if (r.computed != (int)r.tokens.size())
    throw std::logic_error("Scheduler: a token was sampled for a request whose prompt is unread");
  if (is_stop) {
    // The stop token is neither kept nor counted (base/src/engine.cu:926).
    finish(&r, FinishReason::Stop);
    return FinishReason::Stop;
  }
  r.tokens.push_back(token);
  const int generated = (int)r.tokens.size() - r.prompt_len;
  if (generated >= r.max_tokens) { finish(&r, FinishReason::Length); return FinishReason::Length; }
  if ((int)r.tokens.size() >= cfg_.max_model_len) {
    finish(&r, FinishReason::ModelLen);
    return FinishReason::ModelLen;
  }
  return FinishReason::None;
}

void Scheduler::mark_pending(const Plan& plan) {
  for (const PlanEntry& e : plan.entries) {
    if (!e.sample) continue;
    auto it = reqs_.find(e.id);
    if (it == reqs_.end()) continue;
    Req& r = it->second;
    if (r.pending > 1 || r.closing)
      throw std::logic_error("Scheduler: request " + std::to_string(e.id) + " cannot take another pending token");
    if (r.computed != (int)r.tokens.size())
      throw std::logic_error("Scheduler: a token is pending for a request whose prompt is unread");
    r.tokens.push_back(kPendingToken);
    ++r.pending;
    const int generated = (int)r.tokens.size() - r.prompt_len;
    r.closing = generated >= r.max_tokens || (int)r.tokens.size() >= cfg_.max_model_len;
  }
}

FinishReason Scheduler::resolve(int64_t id, int token, bool is_stop) {
  auto it = reqs_.find(id);
  if (it == reqs_.end()) return any(id).reason;   // ended meanwhile
  Req& r = it->second;
  if (!r.pending) throw std::logic_error("Scheduler: request " + std::to_string(id) + " has no pending token");
  const size_t at = r.tokens.size() - r.pending;   // the oldest unknown token
  if (is_stop) {
    // neither the stop token nor anything sampled after it is kept
    r.tokens.resize(at);
    r.pending = 0;
    r.closing = false;
    finish(&r, FinishReason::Stop);
    return FinishReason::Stop;
  }
  r.tokens[at] = token;
  --r.pending;
  if (r.pending) return FinishReason::None;
  r.closing = false;
  const int generated = (int)r.tokens.size() - r.prompt_len;
  if (generated >= r.max_tokens) { finish(&r, FinishReason::Length); return FinishReason::Length; }
  if ((int)r.tokens.size() >= cfg_.max_model_len) {
    finish(&r, FinishReason::ModelLen);
    return FinishReason::ModelLen;
  }
  return FinishReason::None;
}

bool Scheduler::has_pending(int64_t id) const {
  auto it = reqs_.find(id);
  return it != reqs_.end() && it->second.pending > 0;
}

void Scheduler::abort(int64_t id) {
  auto it = reqs_.find(id);
  if (it == reqs_.end()) return;
  finish(&it->second, FinishReason::Aborted);
}

const std::vector<int>& Scheduler::tokens(int64_t id) const { return any(id).tokens; }
int Scheduler::prompt_len(int64_t id) const { return any(id).prompt_len; }
std::vector<int> Scheduler::output(int64_t id) const {
  const Req& r = any(id);
  return std::vector<int>(r.tokens.begin() + r.prompt_len, r.tokens.end() - r.pending);
}
FinishReason Scheduler::finish_reason(int64_t id) const { return any(id).reason; }
int Scheduler::preemptions_of(int64_t id) const { return any(id).preemptions; }

std::vector<int> Scheduler::take_finished(int64_t id) {
  auto it = done_.find(id);
  if (it == done_.end())
    throw std::out_of_range("Scheduler: request " + std::to_string(id) + " has not finished");
  std::vector<int> out(it->second.tokens.begin() + it->second.prompt_len, it->second.tokens.end());
  done_.erase(it);
  return out;
}

}  // namespace kvb
