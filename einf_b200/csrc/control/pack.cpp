// Packing a batch plan into the step buffer (see control.h).
#include <algorithm>

#include "control.h"

namespace einf {

std::vector<StepField> step_layout(int tokens, int requests, int wanted, int groups, int table_width, int tiles,
                                   int single_tokens, int* total) {
  std::vector<StepField> fields;
  int offset = 0;
  auto add = [&](const std::string& name, int count) {
    fields.push_back({name, offset, count});
    offset += (count + 3) / 4 * 4;
  };
  add("status", 1);
  add("token_ids", tokens);
  add("positions", tokens);
  add("seq_of_token", tokens);
  add("q_start", requests + 1);
  add("context_lens", requests);
  add("state_slots", requests);
  add("logit_rows", wanted);
  add("q_tiles", 4 * tiles);
  add("single_tokens", single_tokens);
  for (int g = 0; g < groups; ++g) add("slots" + std::to_string(g), tokens);
  for (int g = 0; g < groups; ++g) add("block_table" + std::to_string(g), requests * table_width);
  if (total) *total = offset;
  return fields;
}

PackedStep pack_step(const std::vector<ScheduledRequest>& requests, const std::vector<std::vector<int>>* want,
                     int32_t* buffer, size_t capacity, const PackConfig& config, int pad_requests_to) {
  if (requests.empty()) throw InvalidArgument("a step needs at least one request");
  const int page = config.page_size;
  const int groups = static_cast<int>(config.pages_per_group.size());
  const int real = static_cast<int>(requests.size());
  if (want && static_cast<int>(want->size()) != real) throw InvalidArgument("want must have one entry per request");
  const int pad = std::max(0, pad_requests_to - real);

  PackedStep out;
  int tokens = 0, wanted = 0, tiles = 0, singles = 0;
  for (int i = 0; i < real; ++i) {
    const int q_len = static_cast<int>(requests[i].input_token_ids.size());
    if (q_len <= 0) throw InvalidArgument("every request of a step brings at least one token");
    tokens += q_len;
    if (q_len == 1) singles += 1;
    else tiles += (q_len + config.q_tile - 1) / config.q_tile;
    wanted += want ? static_cast<int>((*want)[i].size()) : (requests[i].need_sample ? 1 : 0);
  }
  tokens += pad;
  singles += pad;
  wanted += pad;
  const int num_requests = real + pad;
  if (tokens > config.max_tokens)
    throw InvalidArgument("the step has " + std::to_string(tokens) + " tokens, the engine was built for " +
                          std::to_string(config.max_tokens));
  if (num_requests > config.max_requests)
    throw InvalidArgument("the step has " + std::to_string(num_requests) + " requests, the engine was built for " +
                          std::to_string(config.max_requests));
  out.fields = step_layout(tokens, num_requests, wanted, groups, config.table_width, tiles, singles, &out.total);
  if (static_cast<size_t>(out.total) > capacity) throw InvalidArgument("the step buffer is too small for this step");
  auto field = [&](const std::string& name) -> int32_t* {
    for (const StepField& f : out.fields)
      if (f.name == name) return buffer + f.offset;
    throw StateError("no field " + name);
  };
  int32_t* status = field("status");
  int32_t* token_ids = field("token_ids");
  int32_t* positions = field("positions");
  int32_t* seq_of_token = field("seq_of_token");
  int32_t* q_start = field("q_start");
  int32_t* context_lens = field("context_lens");
  int32_t* state_slots = field("state_slots");
  int32_t* logit_rows = field("logit_rows");
  int32_t* q_tiles = field("q_tiles");
  int32_t* single_tokens = field("single_tokens");
  std::vector<int32_t*> slots(groups), tables(groups);
  for (int g = 0; g < groups; ++g) {
    slots[g] = field("slots" + std::to_string(g));
    tables[g] = field("block_table" + std::to_string(g));
    std::fill(tables[g], tables[g] + static_cast<size_t>(num_requests) * config.table_width, -1);
  }
  status[0] = 0;
  q_start[0] = 0;
  int cursor = 0, row_cursor = 0, tile_cursor = 0, single_cursor = 0;
  out.decode_only = true;
  for (int i = 0; i < real; ++i) {
    const ScheduledRequest& r = requests[i];
    const std::string where = "request " + std::to_string(i);
    const int q_len = static_cast<int>(r.input_token_ids.size());
    const int start = r.start_position;
    if (start < 0) throw InvalidArgument(where + ": negative start position");
    const int end = start + q_len;
    if (q_len != 1) out.decode_only = false;
    out.q_lens.push_back(q_len);
    out.starts.push_back(start);
    out.max_q_len = std::max(out.max_q_len, q_len);
    out.max_context_len = std::max(out.max_context_len, end);
    for (int t = 0; t < q_len; ++t) {
      const int token = r.input_token_ids[t];
      if (token < 0 || token >= config.vocab_size)
        throw InvalidArgument(where + ": token id outside the vocabulary of " + std::to_string(config.vocab_size));
      token_ids[cursor + t] = token;
      positions[cursor + t] = start + t;
      seq_of_token[cursor + t] = i;
    }
    q_start[i + 1] = cursor + q_len;
    context_lens[i] = end;
    state_slots[i] = r.state_slot;
    if (q_len == 1) {
      single_tokens[single_cursor++] = cursor;
    } else {
      out.max_portion_start = std::max(out.max_portion_start, start);
      for (int first = 0; first < q_len; first += config.q_tile) {
        int32_t* tile = q_tiles + 4 * tile_cursor++;
        tile[0] = i;
        tile[1] = cursor + first;
        tile[2] = std::min(config.q_tile, q_len - first);
        tile[3] = start + first;
      }
    }
    if (static_cast<int>(r.block_tables.size()) != groups)
      throw InvalidArgument(where + ": " + std::to_string(r.block_tables.size()) + " block tables for " +
                            std::to_string(groups) + " cache groups");
    const int needed_pages = (end + page - 1) / page;
    for (int g = 0; g < groups; ++g) {
      const std::vector<int>& table = r.block_tables[g];
      const int have = static_cast<int>(table.size());
      if (have < needed_pages)
        throw InvalidArgument(where + ": block table of group " + std::to_string(g) + " has " + std::to_string(have) +
                              " pages, " + std::to_string(needed_pages) + " are needed for " + std::to_string(end) +
                              " tokens");
      if (have > config.table_width)
        throw InvalidArgument(where + ": " + std::to_string(have) + " pages exceed the table width " +
                              std::to_string(config.table_width));
      int32_t* row = tables[g] + static_cast<size_t>(i) * config.table_width;
      for (int p = 0; p < have; ++p) {
        if (table[p] >= config.pages_per_group[g])
          throw InvalidArgument(where + ": page id outside the pool of group " + std::to_string(g));
        row[p] = table[p];
      }
      const int window = config.windows[g];
      const int first_key = window > 0 ? std::max(0, start - window + 1) : 0;
      for (int p = first_key / page; p < needed_pages; ++p)
        if (table[p] < 0)
          throw InvalidArgument(where + ": a page it needs in group " + std::to_string(g) +
                                " is missing from its block table");
      for (int t = 0; t < q_len; ++t) {
        const int pos = start + t;
        slots[g][cursor + t] = table[pos / page] * page + pos % page;
      }
    }
    int count = 0;
    if (want) {
      for (int place : (*want)[i]) {
        if (place < 0 || place >= q_len)
          throw InvalidArgument(where + ": wanted place " + std::to_string(place) + " outside its " +
                                std::to_string(q_len) + " tokens");
        logit_rows[row_cursor + count++] = cursor + place;
      }
    } else if (r.need_sample) {
      logit_rows[row_cursor + count++] = cursor + q_len - 1;
    }
    out.rows_of_request.emplace_back(row_cursor, count);
    row_cursor += count;
    cursor += q_len;
  }
  for (int extra = 0; extra < pad; ++extra) {
    const int i = real + extra;
    token_ids[cursor] = 0;
    positions[cursor] = 0;
    seq_of_token[cursor] = i;
    q_start[i + 1] = cursor + 1;
    context_lens[i] = 1;
    state_slots[i] = -1;
    single_tokens[single_cursor++] = cursor;
    for (int g = 0; g < groups; ++g) {
      int32_t* row = tables[g] + static_cast<size_t>(i) * config.table_width;
      std::fill(row, row + config.table_width, 0);   // any valid page: what is read there is never used
      slots[g][cursor] = -1;                          // and nothing is written
    }
    logit_rows[row_cursor++] = cursor;
    out.q_lens.push_back(1);
    out.starts.push_back(0);
    out.max_q_len = std::max(out.max_q_len, 1);
    out.max_context_len = std::max(out.max_context_len, 1);
    cursor += 1;
  }
  out.num_tokens = tokens;
  out.num_requests = num_requests;
  out.num_wanted = wanted;
  out.num_tiles = tiles;
  out.num_single_tokens = singles;
  return out;
}

}  // namespace einf
