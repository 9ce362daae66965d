// Continuous-batching scheduler with chunked prefill and preemption by recompute.
//
// Counterpart of the upstream paged build's admitQueuedRequests / enforcePageBudget /
// preemptSequence / finishSequence (paged_attention/src/engine.cu:294-370,406-454,
// 640-731,792-838), redesigned around one mixed step: every step carries single
// decode tokens of running requests beside portions of prompts, under one token
// budget.  Upstream runs whole prompts in passes of their own and never splits one.
#pragma once

#include <cstdint>
#include <deque>
#include <string>
#include <unordered_map>
#include <vector>

#include "cache_manager.h"

namespace kvb {

struct SchedulerConfig {
  int max_num_seqs = 64;              // requests that hold cache at the same time
  int max_num_batched_tokens = 2048;  // tokens one step may carry
  int max_model_len = 4096;           // prompt plus output, at most
  int max_prefill_chunk = 0;          // 0: only the budget limits a prompt portion
  int max_portions_per_step = 0;      // 0: any number; else at most so many runs of more than one token in a step
};

enum class FinishReason { None = 0, Stop, Length, ModelLen, CacheExhausted, Aborted };
const char* finish_reason_name(FinishReason r);

struct PlanEntry {
  int64_t id = 0;
  int start = 0;            // position of the first token of this portion
  std::vector<int> tokens;  // the tokens to run; kPendingToken stands for a token that was
                            // sampled on the device and has not reached the host yet
  bool sample = false;      // the portion ends at the request's last known token
};

constexpr int kPendingToken = -1;

struct Plan {
  std::vector<PlanEntry> entries;
  std::vector<int64_t> preempted;  // sent back to the queue's front in this call
  std::vector<int64_t> finished;   // ended in this call because the cache cannot hold them
  int num_tokens = 0;
};

struct SchedulerStats {
  int64_t steps = 0, scheduled_tokens = 0, preemptions = 0, recomputed_tokens = 0;
  int64_t finished = 0;
};

class Scheduler {
 public:
  Scheduler(CacheManager* cache, SchedulerConfig cfg);

  // Queues a request (first come, first served).  Throws std::invalid_argument for
  // an empty prompt, a live id, max_tokens < 1, or a prompt that can never run
  // (longer than max_model_len allows, or needing more pages than the pool has).
  void add(int64_t id, std::vector<int> prompt, int max_tokens);

  // Decides the next step and takes the pages it needs.
  Plan schedule();
  // Records that the plan ran: its tokens are in the cache now.
  void commit(const Plan& plan);
  // Gives a sampled entry its new token.  A stop token ends the request and is not
  // kept.  Returns the reason if the request ended, None otherwise.
  FinishReason append_token(int64_t id, int token, bool is_stop);
  // Running one step ahead of the host's knowledge of the tokens.  mark_pending: the
  // committed plan's sampled entries each have a new token on the device whose value
  // the host does not know yet; it takes its place in the sequence as kPendingToken, so
  // that the next schedule() can plan the step that reads it.  A request whose pending
  // token is its last by count (max_tokens, max_model_len) is not scheduled again.
  // resolve: the value has arrived; same result as append_token.  A request that ended
  // in between (abort, cache exhausted) ignores it and returns its own reason.  Values
  // arrive in the order in which the tokens were marked.  schedule() wants at most one
  // token per request pending (two are, for a moment, between mark_pending of one step and
  // resolve of the step before it); a request with a pending token that went back to the
  // queue is admitted again only once the token is known.
  void mark_pending(const Plan& plan);
  FinishReason resolve(int64_t id, int token, bool is_stop);
  bool has_pending(int64_t id) const;
  void abort(int64_t id);

  bool has_unfinished() const { return !running_.empty() || !waiting_.empty(); }
  int num_running() const { return (int)running_.size(); }
  int num_waiting() const { return (int)waiting_.size(); }
  bool is_live(int64_t id) const { return reqs_.count(id) != 0; }
  bool is_finished(int64_t id) const { return done_.count(id) != 0; }

  const std::vector<int>& tokens(int64_t id) const;  // prompt followed by output
  int prompt_len(int64_t id) const;
  std::vector<int> output(int64_t id) const;
  FinishReason finish_reason(int64_t id) const;
  int preemptions_of(int64_t id) const;
  // Forgets a finished request and returns its output.
  std::vector<int> take_finished(int64_t id);

  const SchedulerStats& stats() const { return stats_; }
  const SchedulerConfig& config() const { return cfg_; }

 private:
  struct Req {
    int64_t id = 0;
    int64_t arrival = 0;
    std::vector<int> tokens;
    int prompt_len = 0;
    int max_tokens = 0;
    int computed = 0;
    int preemptions = 0;
    int pending = 0;       // so many kPendingToken at the end of tokens
    bool closing = false;  // the newest pending token is the last one by count
    FinishReason reason = FinishReason::None;
  };
  const Req& any(int64_t id) const;
  void finish(Req* r, FinishReason why);
  void preempt(size_t running_index, Plan* plan);
  int portion(const Req& r, int budget) const;
  // For a request that no preemption can make room for, in a model with a windowed group:
  // the largest halving of `want` whose pages could be taken (they are then in place); 0: none.
  int shrink_to_fit(const Req& r, int want);
  // Whether the pools that keep every key have room for everything `r` holds by now, beside the
  // growth of the running requests (the test for admission while others run).
  bool room_for_all_of(const Req& r) const;

  CacheManager* cache_;
  SchedulerConfig cfg_;
  int64_t arrivals_ = 0;
  std::unordered_map<int64_t, Req> reqs_;  // waiting or running
  std::unordered_map<int64_t, Req> done_;
  std::vector<int64_t> running_;           // in arrival order
  std::deque<int64_t> waiting_;
  SchedulerStats stats_;
};

}  // namespace kvb
