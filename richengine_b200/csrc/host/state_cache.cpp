#include "state_cache.hpp"

#include <algorithm>
#include <stdexcept>

namespace rkb::engine {

StateCache::Class StateCache::classOf(uint64_t block, const State &state) const noexcept {
  if (inUse(block)) return Class::InUse;
  return state.checkpoint ? Class::Checkpoint : Class::Ordinary;
}

void StateCache::publish(uint64_t block, uint64_t bytes, bool checkpoint) {
  if (!block) throw std::invalid_argument("a composite state sits on a KV block");
  auto found = states_.find(block);
  if (found != states_.end()) {
    State &state = found->second; // the copy that is there is reused: the same block is the same content
    const bool disposable = checkpoint && !inUse(block);
    if (state.invalid) { // a condemned entry a reader still pins is taken over by the new publication
      if (state.resident) bytes_ -= state.bytes;
      state.invalid = false;
      state.resident = false;
      state.stored = false;
    }
    state.checkpoint = state.checkpoint && disposable; // an ordinary state stays ordinary
    if (!state.resident) { // a stored state gains its RAM copy (StateCache::publishCompositeState over a disk entry)
      state.resident = true;
      state.bytes = bytes;
      bytes_ += bytes;
    }
    if (!state.pins) state.lastUsed = clock_();
    if (!state.checkpoint && note_) note_(block);
    return;
  }
  // a state in use is reusable: a checkpoint published there is ordinary from the start
  const bool disposable = checkpoint && !inUse(block);
  states_.emplace(block, State{bytes, clock_(), disposable, 0});
  bytes_ += bytes;
  if (!disposable && note_) note_(block);
  adjust_(block, +1, inUse(block) ? +1 : 0);
}

void StateCache::publishStored(uint64_t block, uint64_t bytes, bool checkpoint) {
  if (!block) throw std::invalid_argument("a composite state sits on a KV block");
  if (contains(block)) throw std::logic_error("a block's state is published once");
  const bool disposable = checkpoint && !inUse(block);
  auto found = states_.find(block);
  if (found != states_.end()) { // a condemned entry a reader still pins is taken over by the new publication
    State &state = found->second;
    if (state.resident) bytes_ -= state.bytes;
    state.invalid = false;
    state.resident = false;
    state.stored = true;
    state.bytes = bytes;
    state.checkpoint = state.checkpoint && disposable;
    if (!state.checkpoint && note_) note_(block);
    return;
  }
  State state{bytes, clock_(), disposable, 0};
  state.resident = false;
  state.stored = true;
  states_.emplace(block, state);
  if (!disposable && note_) note_(block);
  adjust_(block, +1, inUse(block) ? +1 : 0);
}

void StateCache::adoptStored(uint64_t block, uint64_t bytes, uint64_t lastUsed, bool checkpoint) {
  if (!block || !bytes) throw std::invalid_argument("an adopted composite state is a stored copy on a KV block");
  if (states_.count(block)) throw std::invalid_argument("adopted composite state has no block of its own");
  State state{bytes, lastUsed, checkpoint, 0};
  state.resident = false;
  state.stored = true;
  states_.emplace(block, state);
  if (!checkpoint && note_) note_(block);
  adjust_(block, +1, 0);
}

std::vector<StateCache::StoredState> StateCache::storedStates() const {
  std::vector<StoredState> found;
  for (const auto &[block, state] : states_)
    if (state.stored && !state.invalid) found.push_back({block, state.bytes, state.lastUsed, state.checkpoint});
  std::sort(found.begin(), found.end(), [](const StoredState &a, const StoredState &b) { return a.block < b.block; });
  return found;
}

bool StateCache::ordinary(uint64_t block) const noexcept {
  auto found = states_.find(block);
  return found != states_.end() && !found->second.invalid && !found->second.checkpoint;
}
uint64_t StateCache::bytes(uint64_t block) const noexcept {
  auto found = states_.find(block);
  return found == states_.end() ? 0 : found->second.bytes;
}

void StateCache::use(uint64_t block) {
  const bool first = ++uses_[block] == 1;
  auto found = states_.find(block);
  if (found == states_.end()) return; // yet to be published: in use from the moment it appears
  found->second.checkpoint = false;
  if (note_) note_(block);
  if (first) adjust_(block, 0, +1);
}
void StateCache::unuse(uint64_t block) {
  auto use = uses_.find(block);
  if (use == uses_.end() || !use->second) throw std::logic_error("the state at this block is not in use");
  if (--use->second) return;
  uses_.erase(use);
  auto found = states_.find(block);
  if (found == states_.end()) return;
  if (!found->second.pins) found->second.lastUsed = clock_(); // the conversation resumes there next
  adjust_(block, 0, -1);
}
std::vector<uint64_t> StateCache::usedStates() const {
  std::vector<uint64_t> blocks;
  for (const auto &[block, count] : uses_)
    if (count && contains(block)) blocks.push_back(block);
  std::sort(blocks.begin(), blocks.end());
  return blocks;
}

void StateCache::pin(uint64_t block) {
  auto found = states_.find(block);
  if (found == states_.end() || found->second.invalid) throw std::out_of_range("no composite state at this block");
  ++found->second.pins;
  if (hold_) hold_(block, true);
}
void StateCache::unpin(uint64_t block) {
  auto found = states_.find(block);
  if (found == states_.end() || !found->second.pins) throw std::logic_error("the state at this block is not pinned");
  if (!--found->second.pins) {
    found->second.lastUsed = clock_();
    if (found->second.invalid) erase(found);
  }
  if (hold_) hold_(block, false);
}

uint64_t StateCache::resumePoint() const noexcept {
  uint64_t best = 0, bestUsed = 0;
  bool bestOrdinary = false;
  for (const auto &[block, state] : states_) {
    if (state.pins || state.invalid || inUse(block) || !state.resident) continue;
    const bool isOrdinary = !state.checkpoint;
    if (!best || (isOrdinary && !bestOrdinary) || (isOrdinary == bestOrdinary && state.lastUsed > bestUsed)) {
      best = block; bestUsed = state.lastUsed; bestOrdinary = isOrdinary;
    }
  }
  return best;
}

std::optional<StateCandidate> StateCache::oldest(Class wanted, uint64_t withheld) const {
  std::optional<StateCandidate> best;
  for (const auto &[block, state] : states_) {
    if (state.pins || state.invalid || !state.resident || block == withheld || classOf(block, state) != wanted) continue;
    if (!best || state.lastUsed < best->lastUsed || (state.lastUsed == best->lastUsed && block < best->block))
      best = StateCandidate{block, state.lastUsed};
  }
  return best;
}
std::optional<StateCandidate> StateCache::checkpointCandidate(bool keepResumePoint) const {
  return oldest(Class::Checkpoint, keepResumePoint ? resumePoint() : 0);
}
std::optional<StateCandidate> StateCache::ordinaryCandidate(bool keepResumePoint) const {
  return oldest(Class::Ordinary, keepResumePoint ? resumePoint() : 0);
}
std::optional<StateCandidate> StateCache::inUseCandidate() const { return oldest(Class::InUse, 0); }

uint32_t StateCache::evictableStates(bool withInUse) const noexcept {
  uint32_t count = 0;
  for (const auto &[block, state] : states_)
    if (!state.pins && !state.invalid && state.resident && (withInUse || !inUse(block))) ++count;
  return count;
}

void StateCache::erase(std::unordered_map<uint64_t, State>::iterator found) {
  const uint64_t block = found->first;
  if (found->second.resident) bytes_ -= found->second.bytes;
  const bool used = inUse(block);
  states_.erase(found);
  adjust_(block, -1, used ? -1 : 0);
}

void StateCache::forget(uint64_t block) {
  auto found = states_.find(block);
  if (found == states_.end()) return;
  // a pinned state leaves too (the block under it is gone): its pins' holds on the block go with it
  for (uint32_t pin = 0; pin < found->second.pins; ++pin)
    if (hold_) hold_(block, false);
  found->second.pins = 0;
  erase(found);
}

void StateCache::invalidate(uint64_t block) {
  auto found = states_.find(block);
  if (found == states_.end() || found->second.invalid) return;
  if (found->second.pins) found->second.invalid = true; // the reader's copy stays until it lets go
  else erase(found);
}

bool StateCache::reclaim(uint64_t block, uint64_t *freed) {
  auto found = states_.find(block);
  if (found == states_.end() || found->second.pins || found->second.invalid || !found->second.resident) return false;
  if (freed) *freed = found->second.bytes;
  bytes_ -= found->second.bytes;
  if (found->second.stored) { // the copy stored elsewhere keeps the state: only the RAM goes
    found->second.resident = false;
    return true;
  }
  const bool used = inUse(block);
  states_.erase(found);
  adjust_(block, -1, used ? -1 : 0);
  return true;
}

} // namespace rkb::engine
