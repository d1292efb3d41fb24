// state_cache.hpp — composite states attached to KV blocks, and what the reclaim policy needs of them.
//
// In the reference a hybrid model's conversation resumes from a "composite state" (target-recurrent + draft-context
// buffers) published at a complete KV block (runtime/engine/cache/StateCache.hpp:137-379, StateCache.cpp). The KV
// path itself does not read those buffers; what couples them to it is the reclaim policy: KV that a state restores
// through is "needed by a state", a state an unfinished request resumes from is "in use" together with the KV
// above it, disposable checkpoints go before ordinary states, and states in use go last
// (runtime/engine/cache/Cache.hpp:549-556, Cache.cpp:451-628). This is that subset: a state is a byte count on a
// block with a class (checkpoint or ordinary), a recency, a use count and where its copies are: in RAM (what the
// reclaim order takes), stored elsewhere by the model (the reference's disk tier for states; its writers, quota and
// persistence are not rebuilt, a stored copy is a flag), or both. A stored copy costs no RAM and is no reclaim
// candidate; it keeps the KV it restores through worth a tier copy.
#pragma once

#include <cstdint>
#include <functional>
#include <optional>
#include <unordered_map>
#include <vector>

namespace rkb::engine {

struct StateCandidate { uint64_t block = 0; uint64_t lastUsed = 0; };

class StateCache final {
public:
  // adjustBelow(block, states, inUse): a state appeared (+1) or went (-1) at `block`, in use or not; the KV index
  // keeps, per block, how many states (in use) sit strictly below it (KvCache::stateBelow / stateInUseBelow).
  using AdjustBelow = std::function<void(uint64_t block, int states, int inUse)>;
  using Clock = std::function<uint64_t()>;
  // noteReusable(block): a reusable (ordinary) state exists at the block now; the KV index remembers it beyond the
  // state's life (KvCache::noteState, called from StateCache::makeOrdinary), so that a later lookup can tell a state
  // that was lost from one that never was.
  using NoteReusable = std::function<void(uint64_t block)>;
  // hold(block, true/false): a pin takes / gives back an active reference on the state's KV block, so that the block
  // is no eviction candidate while a restore reads the state (StateCache::acquireBlock / release: kv_.retainActive,
  // kv_.releaseActive).
  using Hold = std::function<void(uint64_t block, bool held)>;
  StateCache(AdjustBelow adjust, Clock clock, NoteReusable note = {}, Hold hold = {})
      : adjust_(std::move(adjust)), clock_(std::move(clock)), note_(std::move(note)), hold_(std::move(hold)) {}

  // Publishes a RAM copy at a block (StateCache::publishCompositeState), or reuses the one that is there
  // (StateCache::reuseCompositeState: the copy and its size stay, an ordinary boundary upgrades a checkpoint, a
  // checkpoint cannot downgrade an ordinary state, and the recency moves unless a restore pins the state).
  void publish(uint64_t block, uint64_t bytes, bool checkpoint);
  // Publishes a state whose only copy the model stores elsewhere (StateCache::publishStateToDisk). A block's state
  // is published once: a second publication is a logic error.
  void publishStored(uint64_t block, uint64_t bytes, bool checkpoint);
  // A state an earlier process left stored, with the recency and class its label kept (StateCache::adoptDisk).
  void adoptStored(uint64_t block, uint64_t bytes, uint64_t lastUsed, bool checkpoint);
  // Every state with a stored copy: what a persistent tier's labels name (StateCache::relabel / labelDisk).
  struct StoredState { uint64_t block, bytes, lastUsed; bool checkpoint; };
  std::vector<StoredState> storedStates() const;
  bool contains(uint64_t block) const noexcept { auto f = states_.find(block); return f != states_.end() && !f->second.invalid; }
  bool ordinary(uint64_t block) const noexcept;
  uint64_t bytes(uint64_t block) const noexcept;
  bool stateResident(uint64_t block) const noexcept { auto f = states_.find(block); return f != states_.end() && f->second.resident; }
  // An unfinished request resumes from the state at this block, published or yet to be (StateCache::useState):
  // until every use ends the state is in use, and a checkpoint there becomes ordinary.
  void use(uint64_t block);
  void unuse(uint64_t block);
  bool inUse(uint64_t block) const noexcept { auto f = uses_.find(block); return f != uses_.end() && f->second > 0; }
  std::vector<uint64_t> usedStates() const;
  // Pins (a restore in progress): a pinned state is no candidate and holds its KV block; when the last pin goes the
  // state becomes the newest of its class (StateCache::release).
  void pin(uint64_t block);
  void unpin(uint64_t block);

  // The oldest unpinned state of each class (StateCache::checkpointCandidate / ordinaryCandidate / inUseCandidate).
  // keepResumePoint withholds the resume point: the newest unpinned ordinary state, else the newest checkpoint.
  std::optional<StateCandidate> checkpointCandidate(bool keepResumePoint) const;
  std::optional<StateCandidate> ordinaryCandidate(bool keepResumePoint) const;
  std::optional<StateCandidate> inUseCandidate() const;
  uint64_t resumePoint() const noexcept;
  uint32_t evictableStates(bool withInUse) const noexcept;
  // Frees the RAM copy: a state that is stored elsewhere too stays, without it; one that is not goes (the
  // reference's Unwritten::Drop). False when pinned or without a RAM copy. Returns the bytes freed through `freed`.
  bool reclaim(uint64_t block, uint64_t *freed = nullptr);
  // The block leaves the KV index: its state goes with it.
  // A use outlives it: the request that resumes from the block still holds its handle.
  void forget(uint64_t block);
  // The block's content is lost (a failed read): the state is contained no more; while a restore still pins it the
  // entry stays, condemned, and leaves with the last pin (StateCache::invalidate / discardState).
  void invalidate(uint64_t block);
  uint64_t residentBytes() const noexcept { return bytes_; }
  size_t size() const noexcept { return states_.size(); }

private:
  struct State { uint64_t bytes = 0, lastUsed = 0; bool checkpoint = false; uint32_t pins = 0; bool resident = true, stored = false, invalid = false; };
  enum class Class { Checkpoint, Ordinary, InUse };
  Class classOf(uint64_t block, const State &state) const noexcept;
  void erase(std::unordered_map<uint64_t, State>::iterator found);
  std::optional<StateCandidate> oldest(Class wanted, uint64_t withheld) const;

  AdjustBelow adjust_;
  Clock clock_;
  NoteReusable note_;
  Hold hold_;
  std::unordered_map<uint64_t, State> states_;
  std::unordered_map<uint64_t, uint32_t> uses_;
  uint64_t bytes_ = 0;
};

} // namespace rkb::engine
