// Host-side data preparation either side of the forward path: text -> integer minibatch files -> time-major id
// arrays, and integer hypotheses -> text.  Mirrors the reference's input_file_prep (src/input_file_prep.h) and
// file_helper (src/fileHelper.h, src/file_helper_decoder.h); the intermediate files have the reference's format so
// either program can consume the other's.
//
//   force-decode, sequence-to-sequence  integerize_file_nonLM   src/input_file_prep.h:1958-2547
//   force-decode, sequence (-s)         integerize_file_LM      src/input_file_prep.h:2743-2968
//   decode (-k)                         integerize_file_kbest   src/input_file_prep.h:2970-3134
//   ids -> words                        unint_file              src/input_file_prep.h:3137-3205
//   minibatch reader                    file_helper::read_minibatch  src/fileHelper.h:367-518
//   decode input reader                 file_helper_decoder::read_sentence  src/file_helper_decoder.h:75-131
#pragma once
#include <algorithm>
#include <cstdio>
#include <cstdlib>
#include <fstream>
#include <sstream>
#include <string>
#include <unordered_map>
#include <vector>

#include "model_file.hpp"

namespace zrnn {
namespace text {

// ------------------------------------------------------------------------------------------------ vocabulary
struct Vocab {
  ModelFileHeader header;
  std::unordered_map<std::string, int> src, tgt;
  std::unordered_map<int, std::string> src_rev, tgt_rev;

  bool load(const std::string& model_path, std::string* err) {
    ModelFileReader rd;
    if (!rd.open(model_path, &header, err)) return false;
    for (const auto& kv : rd.source_vocab()) { src[kv.second] = kv.first; src_rev[kv.first] = kv.second; }
    for (const auto& kv : rd.target_vocab()) { tgt[kv.second] = kv.first; tgt_rev[kv.first] = kv.second; }
    return true;
  }
  // unknown source words map to the entry "<UNK>" (src/input_file_prep.h:2238-2244); a file without that entry
  // behaves like the reference's operator[] on the map: id 0
  int src_id(const std::string& w) const {
    auto it = src.find(w);
    if (it != src.end()) return it->second;
    it = src.find("<UNK>");
    return it != src.end() ? it->second : 0;
  }
  // unknown target words map to "<UNK>", or to "<UNK>NULL" when the vocabulary has no plain "<UNK>"
  // (src/input_file_prep.h:2315-2325)
  int tgt_id(const std::string& w) const {
    auto it = tgt.find(w);
    if (it != tgt.end()) return it->second;
    it = tgt.find("<UNK>");
    if (it != tgt.end()) return it->second;
    it = tgt.find("<UNK>NULL");
    return it != tgt.end() ? it->second : 0;
  }
};

inline std::vector<std::string> split_ws(const std::string& line) {
  std::vector<std::string> out;
  std::istringstream iss(line);
  std::string w;
  while (iss >> w) out.push_back(w);
  return out;
}

inline bool read_lines(const std::string& path, std::vector<std::string>* out, std::string* err) {
  std::ifstream in(path.c_str());
  if (!in) { *err = "cannot open " + path; return false; }
  std::string s;
  while (std::getline(in, s)) out->push_back(s);
  return true;
}

inline std::vector<int> parse_ints(const std::string& line) {
  std::vector<int> out;
  const char* p = line.c_str();
  for (;;) {
    char* e;
    const long v = strtol(p, &e, 10);
    if (e == p) break;
    out.push_back((int)v);
    p = e;
  }
  return out;
}

// ------------------------------------------------------------------------------------------------ records
// One sentence (pair) as it stands in the integer minibatch file: four padded rows.
struct Record {
  std::vector<int> src;        // reversed source ids, left-padded with -1 (empty for sequence models)
  std::vector<int> minus_two;  // -2 per source word, -1 under the padding (unused at inference)
  std::vector<int> tgt_in;     // 0 y1 .. yn, right-padded with -1
  std::vector<int> tgt_out;    // y1 .. yn 1, right-padded with -1
  int line_no = -1;            // line of the user's file this came from (-1: filler row)
};

struct PrepStats {
  int lines = 0, kept = 0, src_tokens = 0, tgt_tokens = 0, longest_src = 0, longest_tgt = 0, thrown_tokens = 0;
};

static const int kMinibatchMult = 10;  // sort window = minibatch_size * 10 (src/input_file_prep.h:105)

namespace detail {
struct Raw {
  std::vector<std::string> src, tgt;
  int line_no;
  int total_len() const { return (int)(src.size() + tgt.size()); }
};
// sort by total length inside windows of minibatch_size * 10 sentences (src/input_file_prep.h:2191-2204, 2852-2866).
// The reference uses std::sort, whose order among equal lengths is unspecified; this keeps file order for ties.
inline void window_sort(std::vector<Raw>* data, int minibatch) {
  const size_t win = (size_t)minibatch * kMinibatchMult;
  size_t cur = 0;
  auto cmp = [](const Raw& a, const Raw& b) { return a.total_len() < b.total_len(); };
  while (cur < data->size()) {
    if (cur + win <= data->size()) {
      std::stable_sort(data->begin() + cur, data->begin() + cur + win, cmp);
      cur += win;
    } else {
      std::stable_sort(data->begin() + cur, data->end(), cmp);
      break;
    }
  }
}
}  // namespace detail

// ------------------------------------------------------------------------------------------------ force-decode prep
// integerize_file_nonLM: keep pairs with src+1 < L-2 and tgt+1 < L-2; for minibatch != 1 sort in windows and drop the
// sentences that do not fill the last minibatch; reverse the source; pad per minibatch.
inline bool prep_force_decode_nonlm(const Vocab& v, const std::string& src_path, const std::string& tgt_path,
                                    int longest_sent, int minibatch, std::vector<Record>* out, PrepStats* st,
                                    std::string* err) {
  std::vector<std::string> sl, tl;
  if (!read_lines(src_path, &sl, err) || !read_lines(tgt_path, &tl, err)) return false;
  if (sl.size() != tl.size()) { *err = "Input files are not the same length"; return false; }
  std::vector<detail::Raw> data;
  st->lines = (int)tl.size();
  for (size_t i = 0; i < sl.size(); ++i) {
    detail::Raw r;
    r.src = split_ws(sl[i]);
    r.tgt = split_ws(tl[i]);
    r.line_no = (int)i;
    if (!((int)r.src.size() + 1 >= longest_sent - 2 || (int)r.tgt.size() + 1 >= longest_sent - 2)) {
      st->src_tokens += (int)r.src.size();
      st->tgt_tokens += (int)r.tgt.size();
      st->longest_src = std::max(st->longest_src, (int)r.src.size());
      st->longest_tgt = std::max(st->longest_tgt, (int)r.tgt.size());
      data.push_back(std::move(r));
    } else {
      st->thrown_tokens += (int)(r.src.size() + r.tgt.size());
    }
  }
  if (minibatch != 1) detail::window_sort(&data, minibatch);
  if (data.size() % (size_t)minibatch != 0) data.resize(data.size() - data.size() % (size_t)minibatch);
  if (data.empty()) { *err = "file size is zero, could be wrong input file or all lines are above max sent length"; return false; }
  st->kept = (int)data.size();
  out->clear();
  out->reserve(data.size());
  for (const auto& r : data) {
    Record rec;
    rec.line_no = r.line_no;
    for (const auto& w : r.src) rec.src.push_back(v.src_id(w));
    std::reverse(rec.src.begin(), rec.src.end());
    rec.minus_two.assign(rec.src.size(), -2);
    rec.tgt_in.push_back(0);
    for (const auto& w : r.tgt) {
      const int id = v.tgt_id(w);
      rec.tgt_in.push_back(id);
      rec.tgt_out.push_back(id);
    }
    rec.tgt_out.push_back(1);
    out->push_back(std::move(rec));
  }
  for (size_t cur = 0; cur < out->size(); cur += (size_t)minibatch) {
    const size_t end = std::min(out->size(), cur + (size_t)minibatch);
    size_t ms = 0, mt = 0;
    for (size_t i = cur; i < end; ++i) {
      ms = std::max(ms, (*out)[i].src.size());
      mt = std::max(mt, (*out)[i].tgt_in.size());
    }
    for (size_t i = cur; i < end; ++i) {
      Record& r = (*out)[i];
      r.src.insert(r.src.begin(), ms - r.src.size(), -1);
      r.minus_two.insert(r.minus_two.begin(), ms - r.minus_two.size(), -1);
      r.tgt_in.resize(mt, -1);
      r.tgt_out.resize(mt, -1);
    }
  }
  return true;
}

// integerize_file_LM: keep sentences with len+1 < L-2; sort in windows for minibatch != 1; pad every minibatch to its
// longest sentence plus one extra -1 column; complete the last minibatch with all -1 rows.
inline bool prep_force_decode_lm(const Vocab& v, const std::string& tgt_path, int longest_sent, int minibatch,
                                 std::vector<Record>* out, PrepStats* st, std::string* err) {
  std::vector<std::string> tl;
  if (!read_lines(tgt_path, &tl, err)) return false;
  std::vector<detail::Raw> data;
  st->lines = (int)tl.size();
  for (size_t i = 0; i < tl.size(); ++i) {
    detail::Raw r;
    r.tgt = split_ws(tl[i]);
    r.line_no = (int)i;
    if (!((int)r.tgt.size() + 1 >= longest_sent - 2)) {
      st->tgt_tokens += (int)r.tgt.size();
      st->longest_tgt = std::max(st->longest_tgt, (int)r.tgt.size());
      data.push_back(std::move(r));
    } else {
      st->thrown_tokens += (int)r.tgt.size();
    }
  }
  if (data.empty()) { *err = "file size is zero, could be wrong input file or all lines are above max sent length"; return false; }
  if (minibatch != 1) detail::window_sort(&data, minibatch);
  st->kept = (int)data.size();
  out->clear();
  for (const auto& r : data) {
    Record rec;
    rec.line_no = r.line_no;
    rec.tgt_in.push_back(0);
    for (const auto& w : r.tgt) {
      const int id = v.tgt_id(w);
      rec.tgt_in.push_back(id);
      rec.tgt_out.push_back(id);
    }
    rec.tgt_out.push_back(1);
    out->push_back(std::move(rec));
  }
  for (size_t cur = 0; cur < out->size(); cur += (size_t)minibatch) {
    const size_t end = std::min(out->size(), cur + (size_t)minibatch);
    size_t mt = 0;
    for (size_t i = cur; i < end; ++i) mt = std::max(mt, (*out)[i].tgt_in.size());
    for (size_t i = cur; i < end; ++i) {
      (*out)[i].tgt_in.resize(mt + 1, -1);
      (*out)[i].tgt_out.resize(mt + 1, -1);
    }
  }
  const size_t rem = out->size() % (size_t)minibatch;
  if (rem != 0) {
    const size_t width = out->back().tgt_in.size();
    for (size_t i = rem; i < (size_t)minibatch; ++i) {
      Record filler;
      filler.tgt_in.assign(width, -1);
      filler.tgt_out.assign(width, -1);
      out->push_back(std::move(filler));
    }
  }
  return true;
}

// integerize_file_kbest: reverse every source sentence, keep those with len+1 < L-2, map to ids; a legacy model gets
// id 0 in front (src/input_file_prep.h:3108-3110).  kept_lines receives the user's line number of each sentence.
inline bool prep_kbest(const Vocab& v, const std::string& src_path, int longest_sent, bool legacy,
                       std::vector<std::vector<int>>* out, std::vector<int>* kept_lines, PrepStats* st,
                       std::string* err) {
  std::vector<std::string> sl;
  if (!read_lines(src_path, &sl, err)) return false;
  st->lines = (int)sl.size();
  out->clear();
  for (size_t i = 0; i < sl.size(); ++i) {
    std::vector<std::string> w = split_ws(sl[i]);
    if ((int)w.size() + 1 >= longest_sent - 2) { st->thrown_tokens += (int)w.size(); continue; }
    st->src_tokens += (int)w.size();
    st->longest_src = std::max(st->longest_src, (int)w.size());
    std::vector<int> ids;
    if (legacy) ids.push_back(0);
    for (size_t j = w.size(); j-- > 0;) ids.push_back(v.src_id(w[j]));
    out->push_back(std::move(ids));
    if (kept_lines) kept_lines->push_back((int)i);
  }
  st->kept = (int)out->size();
  return true;
}

// ------------------------------------------------------------------------------------------------ integer files
// Every id is followed by one blank, also the last of a line, as the reference writes them
// (src/input_file_prep.h:2432-2468; sequence models: two empty lines, then the target rows, :2934-2955).
inline void write_int_line(std::ostream& os, const std::vector<int>& v) {
  for (int x : v) os << x << ' ';
  os << '\n';
}
inline bool write_minibatch_file(const std::string& path, const std::vector<Record>& recs, std::string* err) {
  std::ofstream os(path.c_str());
  if (!os) { *err = "cannot write " + path; return false; }
  for (const auto& r : recs) {
    write_int_line(os, r.src);
    write_int_line(os, r.minus_two);
    write_int_line(os, r.tgt_in);
    write_int_line(os, r.tgt_out);
  }
  return (bool)os;
}
inline bool read_minibatch_file(const std::string& path, std::vector<Record>* recs, std::string* err) {
  std::vector<std::string> lines;
  if (!read_lines(path, &lines, err)) return false;
  recs->clear();
  for (size_t i = 0; i + 3 < lines.size(); i += 4) {
    Record r;
    r.src = parse_ints(lines[i]);
    r.minus_two = parse_ints(lines[i + 1]);
    r.tgt_in = parse_ints(lines[i + 2]);
    r.tgt_out = parse_ints(lines[i + 3]);
    if (r.tgt_in.size() != r.tgt_out.size()) { *err = "record " + std::to_string(i / 4) + ": target rows differ in length"; return false; }
    recs->push_back(std::move(r));
  }
  return true;
}
inline bool write_kbest_file(const std::string& path, const std::vector<std::vector<int>>& sents, std::string* err) {
  std::ofstream os(path.c_str());
  if (!os) { *err = "cannot write " + path; return false; }
  for (const auto& s : sents) write_int_line(os, s);
  return (bool)os;
}
inline bool read_kbest_file(const std::string& path, std::vector<std::vector<int>>* sents, std::string* err) {
  std::vector<std::string> lines;
  if (!read_lines(path, &lines, err)) return false;
  sents->clear();
  for (const auto& l : lines) sents->push_back(parse_ints(l));
  return true;
}

// What file_helper::read_minibatch hands to the model for rows [first, first + B): time-major ids
// (idx[b + t * B], src/fileHelper.h:480-509).  Rows may come from several of the reference's minibatches (the
// forward path treats columns independently), so sources are left-padded and targets right-padded to the group's
// maxima here; total_target_words counts the target-input ids != -1 (src/Eigen_Util.h:202-241).
struct Minibatch {
  int B = 0, S_max = 0, T = 0;
  std::vector<int> src, tgt_in, tgt_out;
  int target_words = 0;
};
inline Minibatch make_minibatch(const std::vector<Record>& recs, const std::vector<int>& rows) {
  Minibatch mb;
  mb.B = (int)rows.size();
  for (int i : rows) {
    const Record& r = recs[(size_t)i];
    size_t s0 = 0, t1 = r.tgt_in.size();
    while (s0 < r.src.size() && r.src[s0] == -1) ++s0;
    while (t1 > 0 && r.tgt_in[t1 - 1] == -1) --t1;
    mb.S_max = std::max(mb.S_max, (int)(r.src.size() - s0));
    mb.T = std::max(mb.T, (int)t1);
  }
  if (mb.T == 0) mb.T = 1;  // a group of filler rows only
  mb.src.assign((size_t)mb.S_max * mb.B, -1);
  mb.tgt_in.assign((size_t)mb.T * mb.B, -1);
  mb.tgt_out.assign((size_t)mb.T * mb.B, -1);
  for (int b = 0; b < mb.B; ++b) {
    const Record& r = recs[(size_t)rows[b]];
    size_t s0 = 0;
    while (s0 < r.src.size() && r.src[s0] == -1) ++s0;
    const int S = (int)(r.src.size() - s0);
    for (int j = 0; j < S; ++j) mb.src[(size_t)b + (size_t)(mb.S_max - S + j) * mb.B] = r.src[s0 + j];
    for (size_t t = 0; t < r.tgt_in.size() && (int)t < mb.T; ++t) {
      mb.tgt_in[(size_t)b + t * mb.B] = r.tgt_in[t];
      mb.tgt_out[(size_t)b + t * mb.B] = r.tgt_out[t];
      if (r.tgt_in[t] != -1) mb.target_words++;
    }
  }
  return mb;
}

// ------------------------------------------------------------------------------------------------ ids -> words
// unint_file for decoder output: lines that are empty or begin with '-' or a blank are copied, every other line is
// a row of target ids (src/input_file_prep.h:3179-3201).  Ids missing from the vocabulary print as empty words, as
// the reference's operator[] on its map does.
inline std::string unint_line(const Vocab& v, const std::string& line, bool decoder) {
  if (decoder && (line.empty() || line[0] == '-' || line[0] == ' ')) return line;
  const std::vector<int> ids = parse_ints(line);
  std::string out;
  for (size_t i = 0; i < ids.size(); ++i) {
    auto it = v.tgt_rev.find(ids[i]);
    if (it != v.tgt_rev.end()) out += it->second;
    if (i + 1 != ids.size()) out += ' ';
  }
  return out;
}
inline bool unint_file(const Vocab& v, const std::string& in_path, const std::string& out_path, bool decoder,
                       std::string* err) {
  std::vector<std::string> lines;
  if (!read_lines(in_path, &lines, err)) return false;
  std::ofstream os(out_path.c_str());
  if (!os) { *err = "cannot write " + out_path; return false; }
  for (const auto& l : lines) os << unint_line(v, l, decoder) << '\n';
  return (bool)os;
}

}  // namespace text
}  // namespace zrnn
