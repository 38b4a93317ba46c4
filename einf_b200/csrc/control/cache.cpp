// Page pool, state slots and the cache manager.
#include <algorithm>
#include <limits>
#include <set>

#include "control.h"

namespace einf {

// --- PagePool ---------------------------------------------------------------
PagePool::PagePool(int num_pages) {
  if (num_pages <= 0) throw InvalidArgument("a page pool needs at least one page");
  held_.assign(num_pages, 0);
  free_.reserve(num_pages);
  for (int page = num_pages - 1; page >= 0; --page) free_.push_back(page);  // page 0 on top
}

bool PagePool::is_held(int page) const {
  return page >= 0 && page < capacity() && held_[page] != 0;
}

bool PagePool::allocate(int n, std::vector<int>* out) {
  if (n < 0) throw InvalidArgument("cannot allocate a negative number of pages");
  if (n > free_count()) return false;
  for (int i = 0; i < n; ++i) {
    const int page = free_.back();
    free_.pop_back();
    held_[page] = 1;
    out->push_back(page);
  }
  high_water_ = std::max(high_water_, held_count());
  return true;
}

void PagePool::release(const std::vector<int>& pages) {
  std::set<int> seen;
  for (int page : pages) {
    if (page < 0 || page >= capacity())
      throw StateError("page " + std::to_string(page) + " is outside the pool");
    if (!held_[page]) throw StateError("page " + std::to_string(page) + " is freed twice");
    if (!seen.insert(page).second)
      throw StateError("page " + std::to_string(page) + " is named twice in one release");
  }
  // Last page first, so that pages freed together come back in the order they were held: a
  // context reserved in one go then gets a run of consecutive pages again, which the attention
  // kernels fetch with one copy per 128 keys instead of one per page.
  for (auto page = pages.rbegin(); page != pages.rend(); ++page) {
    held_[*page] = 0;
    free_.push_back(*page);
  }
}

// --- SlotPool ---------------------------------------------------------------
SlotPool::SlotPool(int num_slots) {
  if (num_slots < 0) throw InvalidArgument("the number of state slots cannot be negative");
  held_.assign(num_slots, 0);
  for (int slot = num_slots - 1; slot >= 0; --slot) free_.push_back(slot);
}

int SlotPool::take() {
  if (free_.empty()) return -1;
  const int slot = free_.back();
  free_.pop_back();
  held_[slot] = 1;
  return slot;
}

void SlotPool::give_back(int slot) {
  if (slot < 0 || slot >= capacity()) throw StateError("state slot " + std::to_string(slot) + " is outside the pool");
  if (!held_[slot]) throw StateError("state slot " + std::to_string(slot) + " is freed twice");
  held_[slot] = 0;
  free_.push_back(slot);
}

// --- CacheManager -----------------------------------------------------------
CacheManager::CacheManager(std::vector<GroupSpec> groups, int num_state_slots)
    : groups_(std::move(groups)), slots_(num_state_slots) {
  if (groups_.empty()) throw InvalidArgument("a cache manager needs at least one group");
  for (const GroupSpec& spec : groups_) {
    if (spec.page_size <= 0) throw InvalidArgument("page_size must be positive");
    if (spec.window < 0) throw InvalidArgument("window must not be negative");
    pools_.emplace_back(spec.num_pages);
  }
}

std::vector<RequestId> CacheManager::holders() const {
  std::vector<RequestId> ids;
  for (const auto& item : entries_) ids.push_back(item.first);
  return ids;
}

int CacheManager::first_needed_page(const GroupSpec& spec, int start) const {
  if (spec.window <= 0) return 0;
  // The query at position `start` sees keys start - window + 1 .. start.
  const int first_key = std::max(0, start - spec.window + 1);
  return first_key / spec.page_size;
}

std::vector<int> CacheManager::pages_needed(const RequestId& id, int start, int end) const {
  if (start < 0 || end < start) throw InvalidArgument("bad token range");
  std::vector<int> needed(groups_.size(), 0);
  if (end == start) return needed;
  auto found = entries_.find(id);
  for (size_t g = 0; g < groups_.size(); ++g) {
    const GroupSpec& spec = groups_[g];
    const int first = first_needed_page(spec, start);
    const int last = (end - 1) / spec.page_size;
    int count = 0;
    for (int page = first; page <= last; ++page) {
      const bool have = found != entries_.end() &&
                        page < static_cast<int>(found->second.tables[g].size()) &&
                        found->second.tables[g][page] >= 0;
      if (!have) ++count;
    }
    needed[g] = count;
  }
  return needed;
}

bool CacheManager::room_for(int context_len, int portion) const {
  for (size_t g = 0; g < groups_.size(); ++g) {
    const GroupSpec& spec = groups_[g];
    int tokens = context_len;
    if (spec.window > 0) tokens = std::min(tokens, spec.window + portion);
    int pages = (tokens + spec.page_size - 1) / spec.page_size;
    if (spec.window > 0 && tokens < context_len) {
      // a window rarely starts on a page edge; but it never spans more pages than the whole context
      pages = std::min(pages + 1, (context_len + spec.page_size - 1) / spec.page_size);
    }
    if (pages > pools_[g].free_count()) return false;
  }
  if (slots_.capacity() > 0 && slots_.free_count() == 0) return false;
  return true;
}

bool CacheManager::reserve(const RequestId& id, int start, int end, int* short_group) {
  const std::vector<int> needed = pages_needed(id, start, end);
  auto found = entries_.find(id);
  const bool fresh = found == entries_.end();
  // Check everything before taking anything.
  for (size_t g = 0; g < groups_.size(); ++g) {
    if (needed[g] > pools_[g].free_count()) {
      if (short_group) *short_group = static_cast<int>(g);
      return false;
    }
  }
  if (fresh && slots_.capacity() > 0 && slots_.free_count() == 0) {
    if (short_group) *short_group = -1;
    return false;
  }
  if (fresh) {
    Entry entry;
    entry.tables.resize(groups_.size());
    if (slots_.capacity() > 0) entry.state_slot = slots_.take();
    found = entries_.emplace(id, std::move(entry)).first;
  }
  if (end == start) return true;
  for (size_t g = 0; g < groups_.size(); ++g) {
    const GroupSpec& spec = groups_[g];
    std::vector<int>& table = found->second.tables[g];
    const int first = first_needed_page(spec, start);
    const int last = (end - 1) / spec.page_size;
    if (static_cast<int>(table.size()) <= last) table.resize(last + 1, -1);
    std::vector<int> fresh_pages;
    pools_[g].allocate(needed[g], &fresh_pages);
    size_t next = 0;
    for (int page = first; page <= last; ++page) {
      if (table[page] < 0) table[page] = fresh_pages[next++];
    }
  }
  return true;
}

int CacheManager::advance(const RequestId& id, int cached_len) {
  auto found = entries_.find(id);
  if (found == entries_.end()) return 0;
  int freed = 0;
  for (size_t g = 0; g < groups_.size(); ++g) {
    const GroupSpec& spec = groups_[g];
    if (spec.window <= 0) continue;
    // The next query stands at `cached_len` and needs keys from cached_len - window + 1 on.
    const int first_needed_key = cached_len - spec.window + 1;
    if (first_needed_key <= 0) continue;
    std::vector<int>& table = found->second.tables[g];
    const int whole_pages_passed = std::min<int>(first_needed_key / spec.page_size, static_cast<int>(table.size()));
    std::vector<int> passed;
    for (int page = 0; page < whole_pages_passed; ++page) {
      if (table[page] >= 0) {
        passed.push_back(table[page]);
        table[page] = -1;
      }
    }
    pools_[g].release(passed);
    freed += static_cast<int>(passed.size());
  }
  return freed;
}

void CacheManager::release(const RequestId& id) {
  auto found = entries_.find(id);
  if (found == entries_.end()) return;
  for (size_t g = 0; g < groups_.size(); ++g) {
    std::vector<int> pages;
    for (int page : found->second.tables[g])
      if (page >= 0) pages.push_back(page);
    pools_[g].release(pages);
  }
  if (found->second.state_slot >= 0) slots_.give_back(found->second.state_slot);
  entries_.erase(found);
}

const std::vector<int>& CacheManager::block_table(const RequestId& id, int g) const {
  auto found = entries_.find(id);
  if (found == entries_.end()) throw InvalidArgument("request '" + id + "' holds no cache");
  return found->second.tables.at(g);
}

int CacheManager::state_slot(const RequestId& id) const {
  auto found = entries_.find(id);
  return found == entries_.end() ? -1 : found->second.state_slot;
}

long long CacheManager::capacity_tokens() const {
  long long best = std::numeric_limits<long long>::max();
  for (const GroupSpec& spec : groups_) {
    if (spec.window > 0) continue;  // a windowed group bounds the window, not the length
    best = std::min(best, static_cast<long long>(spec.num_pages) * spec.page_size);
  }
  return best;
}

void CacheManager::check_invariants() const {
  for (size_t g = 0; g < groups_.size(); ++g) {
    std::vector<int> owners(pools_[g].capacity(), 0);
    for (const auto& item : entries_) {
      for (int page : item.second.tables[g]) {
        if (page < 0) continue;
        if (page >= pools_[g].capacity()) throw StateError("a block table names a page outside the pool");
        if (++owners[page] > 1) throw StateError("page " + std::to_string(page) + " is held twice");
        if (!pools_[g].is_held(page)) throw StateError("page " + std::to_string(page) + " is in a table but free");
      }
    }
    int held = 0;
    for (int count : owners) held += count;
    if (held != pools_[g].held_count())
      throw StateError("group " + std::to_string(g) + ": " + std::to_string(pools_[g].held_count() - held) +
                       " page(s) are held by no request");
  }
  std::set<int> slots;
  for (const auto& item : entries_) {
    if (item.second.state_slot >= 0 && !slots.insert(item.second.state_slot).second)
      throw StateError("a state slot is held twice");
  }
  if (static_cast<int>(slots.size()) != slots_.capacity() - slots_.free_count())
    throw StateError("a state slot is held by no request");
}

}  // namespace einf
