#include "scheduler.hpp"

#include <algorithm>
#include <cmath>

namespace ferrum {

Scheduler::Scheduler(CacheManager* cache, SchedulerConfig cfg) : cache_(cache), cfg_(cfg) {
  if (!cache_) throw SchedulerError("scheduler: no cache manager");
  cfg_.max_batch_tokens = std::max(1, cfg_.max_batch_tokens);  // crates/scheduler/src/batcher.rs:48
  cfg_.max_batch_seqs = std::max(1, std::min(cfg_.max_batch_seqs, cache_->max_requests()));
  const long long cap = cache_->capacity_tokens();
  if (cfg_.max_model_len <= 0 || cfg_.max_model_len > cap) cfg_.max_model_len = (int)std::min<long long>(cap, 1 << 30);
}

void Scheduler::submit(uint64_t id, std::vector<int32_t> prompt, int max_new_tokens, float temperature, float top_p,
                       uint64_t seed, std::vector<int32_t> stop) {
  if (prompt.empty()) throw InvalidRequest("prompt must not be empty");
  if (!(temperature >= 0.0f) || !std::isfinite(temperature)) throw InvalidRequest("temperature must be finite and >= 0");
  if (!(top_p > 0.0f && top_p <= 1.0f)) throw InvalidRequest("top_p must be in (0, 1]");
  if (temperature > 0.0f && top_p != 1.0f) throw InvalidRequest("top_p other than 1 is not implemented");
  if (max_new_tokens < 0) throw InvalidRequest("max_new_tokens must not be negative");
  if (cfg_.n_vocab > 0)
    for (auto t : prompt)
      if (t < 0 || t >= cfg_.n_vocab) throw InvalidRequest("prompt token id is outside the vocabulary");
  if ((long long)prompt.size() + max_new_tokens > cfg_.max_model_len)
    throw InvalidRequest("prompt plus max_new_tokens exceeds what the cache can hold for one request (" +
                         std::to_string(cfg_.max_model_len) + " tokens)");
  for (auto& s : queue_)
    if (s.id == id) throw InvalidRequest("request id is already queued");
  for (auto& s : active_)
    if (s.id == id) throw InvalidRequest("request id is already running");
  Seq s;
  s.id = id;
  s.prompt_len = (int)prompt.size();
  s.tokens = std::move(prompt);
  s.max_new = max_new_tokens;
  s.temperature = temperature;
  s.seed = seed;
  s.stop = std::move(stop);
  queue_.push_back(std::move(s));
}

void Scheduler::cancel(uint64_t id) {
  if (!ahead_.empty()) throw SchedulerError("cancel between plan_ahead and commit");
  // a planned row of the request is void from here on: the batch may be running already, what it
  // computes for the row is ignored (pages it frees are handed out to later steps only)
  for (auto& e : plan_)
    if (e.id == id) e.slot = -1;
  for (auto it = queue_.begin(); it != queue_.end(); ++it)
    if (it->id == id) {
      queue_.erase(it);
      return;
    }
  for (size_t i = 0; i < active_.size(); ++i)
    if (active_[i].id == id) {
      cache_->close(active_[i].slot);
      active_.erase(active_.begin() + i);
      return;
    }
  throw NotFound("request not found");
}

bool Scheduler::admit_one() {
  if (queue_.empty() || (int)active_.size() >= cfg_.max_batch_seqs || cache_->free_slots() == 0) return false;
  const Seq& next = queue_.front();
  int first = std::min(next.prompt_len, cfg_.max_batch_tokens);
  if (cfg_.chunk_size > 0) first = std::min(first, cfg_.chunk_size);
  int decoding = 0;
  for (auto& s : active_) decoding += s.decoding;
  for (int g = 0; g < cache_->n_groups(); ++g) {
    const int ps = cache_->group(g).page_size;
    const int need = (first + ps - 1) / ps;
    // leave one page per decoding sequence so that admission does not starve them at once
    if (cache_->free_pages(g) < need + decoding) return false;
  }
  Seq s = std::move(queue_.front());
  queue_.pop_front();
  s.slot = cache_->open();
  s.cursor = 0;
  s.decoding = false;
  s.admitted_at = ++clock_;
  active_.push_back(std::move(s));
  return true;
}

int Scheduler::preempt_youngest() {
  if (active_.empty()) throw SchedulerError("preempt without an active sequence");
  size_t v = 0;
  for (size_t i = 1; i < active_.size(); ++i)
    if (active_[i].admitted_at > active_[v].admitted_at) v = i;
  Seq s = std::move(active_[v]);
  active_.erase(active_.begin() + v);
  // a portion already planned for it in this step is withdrawn
  plan_.erase(std::remove_if(plan_.begin(), plan_.end(), [&](const PlanEntry& e) { return e.id == s.id; }), plan_.end());
  cache_->close(s.slot);
  s.slot = -1;
  s.cursor = 0;
  s.decoding = false;
  s.prompt_len = (int)s.tokens.size();  // recompute everything it has seen and said
  ++stats_.preemptions;
  queue_.push_front(std::move(s));
  return (int)v;
}

std::vector<PlanEntry> Scheduler::plan() {
  if (planned_) throw SchedulerError("plan called twice without commit or abandon");
  plan_.clear();
  while (admit_one()) {
  }
  for (int attempt = 0; attempt < 1 + cache_->max_requests(); ++attempt) {
    int budget = cfg_.max_batch_tokens;
    plan_.clear();
    // ---- one token for every decoding sequence, in active order (batcher.rs:132-186)
    std::vector<uint64_t> decode_ids;
    for (auto& s : active_)
      if (s.decoding) decode_ids.push_back(s.id);
    for (uint64_t id : decode_ids) {
      if (budget == 0) break;
      bool gone = false;
      size_t idx = 0;
      for (;;) {
        idx = active_.size();
        for (size_t i = 0; i < active_.size(); ++i)
          if (active_[i].id == id) idx = i;
        if (idx == active_.size()) {
          gone = true;
          break;
        }
        if (cache_->can_grow(active_[idx].slot, active_[idx].cursor + 1)) break;
        const size_t before = plan_.size();
        preempt_youngest();
        budget += (int)(before - plan_.size());  // a withdrawn decode entry gives its token back
      }
      if (gone) continue;
      Seq& s = active_[idx];
      cache_->grow(s.slot, s.cursor + 1);
      plan_.push_back(PlanEntry{s.id, s.slot, s.cursor, {s.tokens.back()}, true, s.temperature, s.seed, s.generated});
      --budget;
    }
    // ---- prompt portions with what is left of the budget, oldest first (batcher.rs:191-255)
    for (size_t i = 0; i < active_.size() && budget > 0; ++i) {
      Seq& s = active_[i];
      if (s.decoding) continue;
      const int remaining = s.prompt_len - s.cursor;
      if (remaining <= 0) continue;
      int take = std::min(budget, remaining);
      if (cfg_.chunk_size > 0) take = std::min(take, cfg_.chunk_size);
      take = cache_->max_growable(s.slot, s.cursor + take) - s.cursor;
      if (take <= 0) break;  // no page for it now; later prompts do not overtake it
      cache_->grow(s.slot, s.cursor + take);
      PlanEntry e{s.id, s.slot, s.cursor, {}, false, s.temperature, s.seed, s.generated};
      e.tokens.assign(s.tokens.begin() + s.cursor, s.tokens.begin() + s.cursor + take);
      e.sample = (s.cursor + take == s.prompt_len) && s.max_new > 0;
      plan_.push_back(std::move(e));
      budget -= take;
    }
    if (!plan_.empty() || active_.empty()) break;
    // nothing can run although sequences are active: they hold each other's pages
    if (active_.size() == 1) {
      // alone and still without room: it can never finish; end it rather than spin
      pending_.push_back(Event{1, active_[0].id, -1, FINISH_LENGTH});
      finish(0);
      while (admit_one()) {
      }
      if (active_.empty()) break;
      continue;
    }
    preempt_youngest();
  }
  planned_ = !plan_.empty();
  return plan_;
}

void Scheduler::finish(size_t idx) {
  cache_->close(active_[idx].slot);
  active_.erase(active_.begin() + idx);
  ++stats_.finished;
}

void Scheduler::abandon() {
  plan_.clear();
  ahead_.clear();
  planned_ = false;
}

std::vector<PlanEntry> Scheduler::plan_ahead() {
  if (!planned_ || !ahead_.empty() || !pending_.empty() || !queue_.empty()) return {};
  // where every active sequence stands once the current plan is committed, if nothing stops
  struct After {
    int cursor;
    bool decoding, samples_now;
  };
  std::vector<After> after(active_.size());
  for (size_t i = 0; i < active_.size(); ++i) after[i] = After{active_[i].cursor, active_[i].decoding, false};
  std::vector<size_t> sampled_seq;   // the sequences of this step's sampled rows, in its order
  for (auto& e : plan_) {
    if (e.slot < 0) return {};
    size_t idx = active_.size();
    for (size_t i = 0; i < active_.size(); ++i)
      if (active_[i].id == e.id) idx = i;
    if (idx == active_.size()) return {};
    const Seq& s = active_[idx];
    const int len_after = e.pos0 + (int)e.tokens.size();
    after[idx].cursor = len_after;
    if (e.sample) {
      if (s.generated + 1 >= s.max_new) return {};  // this step's token is its last: the batch changes
      if (len_after + 1 > cfg_.max_model_len) return {};
      after[idx].decoding = true;
      after[idx].samples_now = true;
      sampled_seq.push_back(idx);
    } else if (len_after >= s.prompt_len) {
      return {};  // a prompt ends without a token (nothing to generate): the sequence finishes at commit
    }
  }
  // a decoding sequence that sits this step out knows its token already: the ordinary plan takes it
  for (size_t i = 0; i < active_.size(); ++i)
    if (active_[i].decoding && !after[i].samples_now) return {};
  int budget = cfg_.max_batch_tokens;
  if ((int)sampled_seq.size() > budget) return {};
  // pages: one more position for every sampled row, without preemption
  std::vector<int> need(cache_->n_groups(), 0);
  for (size_t idx : sampled_seq) {
    const auto miss = cache_->pages_missing(active_[idx].slot, after[idx].cursor + 1);
    for (size_t g = 0; g < miss.size(); ++g) need[g] += miss[g];
  }
  for (size_t g = 0; g < need.size(); ++g)
    if (need[g] > cache_->free_pages((int)g)) return {};  // the ordinary plan decides who is preempted
  for (size_t idx : sampled_seq) {
    const Seq& s = active_[idx];
    cache_->grow(s.slot, after[idx].cursor + 1);
    PlanEntry e{s.id, s.slot, after[idx].cursor, {-1}, true, s.temperature, s.seed, s.generated + 1};
    e.from_device = true;
    ahead_.push_back(std::move(e));
    --budget;
  }
  // portions of the prompts that are not done, oldest first, as plan() hands them out
  for (size_t i = 0; i < active_.size() && budget > 0; ++i) {
    const Seq& s = active_[i];
    if (after[i].decoding) continue;
    const int remaining = s.prompt_len - after[i].cursor;
    if (remaining <= 0) continue;
    int take = std::min(budget, remaining);
    if (cfg_.chunk_size > 0) take = std::min(take, cfg_.chunk_size);
    take = cache_->max_growable(s.slot, after[i].cursor + take) - after[i].cursor;
    if (take <= 0) break;  // no page for it now; later prompts do not overtake it
    cache_->grow(s.slot, after[i].cursor + take);
    PlanEntry e{s.id, s.slot, after[i].cursor, {}, false, s.temperature, s.seed, s.generated};
    e.tokens.assign(s.tokens.begin() + after[i].cursor, s.tokens.begin() + after[i].cursor + take);
    e.sample = (after[i].cursor + take == s.prompt_len) && s.max_new > 0;
    ahead_.push_back(std::move(e));
    budget -= take;
  }
  return ahead_;
}

std::vector<Event> Scheduler::commit(const std::vector<int32_t>& sampled) {
  std::vector<Event> events;
  events.swap(pending_);
  if (!planned_) {
    if (!sampled.empty()) throw SchedulerError("commit without a plan");
    return events;
  }
  size_t want = 0;
  for (auto& e : plan_) want += e.sample;
  if (sampled.size() != want) throw SchedulerError("commit: number of sampled tokens does not match the plan");
  if (cfg_.n_vocab > 0)
    for (auto t : sampled)
      if (t < 0 || t >= cfg_.n_vocab) throw SchedulerError("commit: sampled token id is outside the vocabulary");
  ++stats_.steps;
  size_t k = 0;
  for (auto& e : plan_) {
    if (e.slot < 0) {  // void row of a batch planned ahead: its sequence ended before the batch was read
      k += e.sample;
      continue;
    }
    size_t idx = active_.size();
    for (size_t i = 0; i < active_.size(); ++i)
      if (active_[i].id == e.id) idx = i;
    if (idx == active_.size()) throw SchedulerError("commit: planned sequence is not active");
    Seq& s = active_[idx];
    const int n = (int)e.tokens.size();
    cache_->commit(s.slot, e.pos0 + n);
    s.cursor = e.pos0 + n;
    if (s.decoding) stats_.decode_tokens += n; else stats_.prompt_tokens += n;
    if (!s.decoding && s.cursor < s.prompt_len) continue;  // more of the prompt to come
    if (!e.sample) {
      // prompt done and nothing to generate (batcher.rs:238-248)
      events.push_back(Event{1, s.id, -1, FINISH_LENGTH});
      finish(idx);
      continue;
    }
    // emit_generated (batcher.rs:257-288)
    const int32_t next = sampled[k++];
    s.generated += 1;
    s.tokens.push_back(next);
    s.decoding = true;
    events.push_back(Event{0, s.id, next, 0});
    const bool stop = std::find(s.stop.begin(), s.stop.end(), next) != s.stop.end() ||
                      std::find(cfg_.eos_token_ids.begin(), cfg_.eos_token_ids.end(), next) != cfg_.eos_token_ids.end();
    if (stop || s.generated >= s.max_new) {
      events.push_back(Event{1, s.id, -1, stop ? FINISH_STOP : FINISH_LENGTH});
      finish(idx);
    }
  }
  plan_.clear();
  planned_ = false;
  if (!ahead_.empty()) {
    // the batch planned ahead is the current one now; rows of sequences that ended are void
    for (auto& a : ahead_) {
      size_t idx = active_.size();
      for (size_t i = 0; i < active_.size(); ++i)
        if (active_[i].id == a.id) idx = i;
      if (idx == active_.size()) a.slot = -1;
      else if (a.from_device) a.tokens[0] = active_[idx].tokens.back();
    }
    plan_.swap(ahead_);
    ahead_.clear();
    planned_ = true;
  }
  return events;
}

}  // namespace ferrum
