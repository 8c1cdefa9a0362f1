// Continuous batcher: admits requests, cuts prompts into portions under a token budget,
// decodes, finishes and frees, and decides what happens when pages run out.
//
// It follows the reference's batcher (crates/scheduler/src/batcher.rs): a FIFO queue and an
// active list; every step first gives each decoding sequence one token, then spends what is
// left of the budget on prompt portions; the first generated token is sampled from the last
// row of the final portion in the same step (:233-236); a stopping token is emitted before
// the sequence finishes (:257-288); max_new_tokens == 0 finishes with Length and no token
// (:238-248).  Differences: one step is ONE batch for the model (plan -> run -> commit), not
// one forward call per sequence; several prompts may get a portion in the same step; and
// temperature sampling is accepted.
//
// A step may be planned one ahead: between plan() and commit(), plan_ahead() gives the batch that
// follows if no sampled row draws a stopping token, so that the engine can put it on the GPU's
// queue before it has read the current step's tokens.  Its rows: first one token for every row
// that samples in the current step, in that step's order (their ids are not known yet: the GPU
// hands them from one step to the next), then the next portions of prompts that are not done.
// commit() then turns it into the current plan; a row whose sequence did stop (or was cancelled)
// is void: its slot is -1, the GPU computes it for nothing and its sampled id is ignored.
//
// When pages run out: a decoding sequence that needs a page takes it from the most recently
// admitted running sequence, which is preempted: its pages and slot are freed and it goes
// back to the head of the queue with prompt := prompt + tokens generated so far, to be
// recomputed later (the reference's restore_kv replays a prefix from position 0 in the same
// spirit, :291-327).  Tokens already emitted stay emitted.  A prompt portion never preempts;
// it shrinks to the pages that are free, or waits.  If nothing at all can run, the youngest
// sequence is preempted so that the oldest can.
#pragma once
#include <cstdint>
#include <deque>
#include <string>
#include <vector>

#include "cache_manager.hpp"

namespace ferrum {

struct InvalidRequest : std::runtime_error { using std::runtime_error::runtime_error; };
struct NotFound : std::runtime_error { using std::runtime_error::runtime_error; };
struct SchedulerError : std::runtime_error { using std::runtime_error::runtime_error; };

enum FinishReason : int { FINISH_STOP = 0, FINISH_LENGTH = 1, FINISH_CANCELLED = 2 };

struct SchedulerConfig {
  int max_batch_tokens = 2048;   // token budget of a step (>= 1)
  int max_batch_seqs = 256;      // sequences that may be active at once
  int chunk_size = 0;            // cap on one prompt portion; 0 = none
  int max_model_len = 0;         // prompt + new tokens may not exceed this; 0 = cache capacity
  int n_vocab = 0;               // token ids must be below this; 0 = unchecked
  std::vector<int32_t> eos_token_ids;  // ids that end a sequence with reason Stop; empty: the model names none
};

struct PlanEntry {
  uint64_t id;
  int slot;
  int pos0;                      // positions pos0 .. pos0 + tokens.size() - 1
  std::vector<int32_t> tokens;
  bool sample;                   // the last of these tokens yields the next token
  float temperature;
  uint64_t seed;
  int counter;                   // tokens generated before this one (keys the random draw)
  bool from_device = false;      // plan_ahead: the one token is the id the step before draws for this row (-1 here)
};

struct Event {
  int kind;                      // 0 = token, 1 = finished
  uint64_t id;
  int32_t token;
  int reason;
};

struct SchedulerStats {
  uint64_t steps = 0, prompt_tokens = 0, decode_tokens = 0, preemptions = 0, finished = 0;
};

class Scheduler {
 public:
  Scheduler(CacheManager* cache, SchedulerConfig cfg);

  void submit(uint64_t id, std::vector<int32_t> prompt, int max_new_tokens, float temperature, float top_p,
              uint64_t seed, std::vector<int32_t> stop);
  // Removes a queued or running request and frees what it holds; emits no event.
  void cancel(uint64_t id);

  // Decide this step's batch and reserve its pages.  Empty when nothing can run.
  std::vector<PlanEntry> plan();
  // The batch ran; `sampled` has one id per entry with sample == true, in plan order.
  std::vector<Event> commit(const std::vector<int32_t>& sampled);
  // The batch did not run: forget the plan, every sequence is as before the step.
  void abandon();
  // Between plan() and commit(): the next step's batch, if it is decided already whatever tokens
  // this step draws short of a stopping token: every row that samples has tokens left to
  // generate, nothing is queued, every decoding sequence is in the plan, no prompt ends without
  // a token, and pages suffice without preemption.  Its pages are reserved.  The entries with
  // from_device come first, one per sampled row of this step in the same order, each with the
  // one token id -1; portions of unfinished prompts follow.  Empty when the next batch cannot be
  // told yet.
  std::vector<PlanEntry> plan_ahead();
  bool planned() const { return planned_; }

  int queued() const { return (int)queue_.size(); }
  int active() const { return (int)active_.size(); }
  bool idle() const { return queue_.empty() && active_.empty(); }
  const SchedulerStats& stats() const { return stats_; }

 private:
  struct Seq {
    uint64_t id = 0;
    std::vector<int32_t> tokens;  // prompt followed by generated tokens
    int prompt_len = 0;           // tokens to prefill before sampling starts (grows on preemption)
    int cursor = 0;               // tokens whose keys are in the cache
    int generated = 0;
    int max_new = 0;
    float temperature = 0.f;
    uint64_t seed = 0;
    std::vector<int32_t> stop;
    bool decoding = false;
    int slot = -1;
    uint64_t admitted_at = 0;
  };
  bool admit_one();
  // Preempts the most recently admitted active sequence; returns its index before removal.
  int preempt_youngest();
  void finish(size_t idx);

  CacheManager* cache_;
  SchedulerConfig cfg_;
  std::deque<Seq> queue_;
  std::vector<Seq> active_;
  std::vector<PlanEntry> plan_;
  std::vector<PlanEntry> ahead_;  // plan_ahead()'s batch until commit() makes it the plan
  std::vector<Event> pending_;   // events decided while planning, delivered by the next commit
  bool planned_ = false;
  uint64_t clock_ = 0;
  SchedulerStats stats_;
};

}  // namespace ferrum
