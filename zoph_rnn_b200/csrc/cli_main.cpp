// Command-line front end for the inference paths of the reference program (src/main.cu):
//   --force-decode / -f   per-minibatch log-probabilities and perplexity     (src/main.cu:1097-1201, 1538-1560)
//   --decode / -k         beam-search k-best decoding                          (src/main.cu:955-1095, 1575-1615)
// It accepts the reference's flags with the reference's meaning and file formats, prepares the integer files the
// way input_file_prep does, runs every minibatch through the C-ABI library and writes the reference's outputs.
// Training flags are recognised and refused.  The binary contains no device code: all work goes through zrnn.h.
#include <sys/stat.h>
#include <sys/wait.h>
#include <unistd.h>

#include <algorithm>
#include <chrono>
#include <cmath>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <fstream>
#include <iomanip>
#include <iostream>
#include <map>
#include <numeric>
#include <set>
#include <string>
#include <vector>

#include "../../include/zrnn.h"
#include "text_data.hpp"

namespace {

using zrnn::text::Minibatch;
using zrnn::text::PrepStats;
using zrnn::text::Record;
using zrnn::text::Vocab;

// ------------------------------------------------------------------------------------------------ logging
// BZ_CUDA::logger (src/logger.h): everything printed to the terminal also goes to --logfile.
struct Logger {
  std::ofstream file;
  template <class T>
  Logger& operator<<(const T& x) {
    std::cout << x;
    if (file.is_open()) file << x;
    return *this;
  }
  void flush() {
    std::cout.flush();
    if (file.is_open()) file.flush();
  }
};
Logger logger;

[[noreturn]] void die(const std::string& msg) {
  logger << "ERROR: " << msg << "\n";
  logger.flush();
  exit(EXIT_FAILURE);
}

// ------------------------------------------------------------------------------------------------ options
// The reference declares its options with boost::program_options (src/main.cu:127-262): `arity` 0 = switch,
// 1 = one value, 2 = multitoken.  `scope`: 'i' used by the inference paths, 't' training only (refused),
// 'x' inference options of features that are not part of this program (refused with the reason).
struct OptSpec {
  const char* name;
  char short_name;
  int arity;
  char scope;
};
const OptSpec kOptions[] = {
    {"help", 'h', 0, 'i'},
    {"force-decode", 'f', 2, 'i'},
    {"decode", 'k', 2, 'i'},
    {"decode-main-data-files", 0, 2, 'i'},
    {"sequence", 's', 0, 'i'},
    {"beam-size", 'b', 1, 'i'},
    {"penalty", 'p', 1, 'i'},
    {"print-score", 0, 1, 'i'},
    {"dec-ratio", 0, 2, 'i'},
    {"longest-sent", 'L', 1, 'i'},
    {"minibatch-size", 'm', 1, 'i'},
    {"multi-gpu", 'M', 2, 'i'},
    {"tmp-dir-location", 0, 1, 'i'},
    {"logfile", 0, 1, 'i'},
    {"attention-width", 0, 1, 'i'},
    {"legacy-model", 0, 1, 'i'},
    {"UNK-decode", 0, 1, 'i'},
    // accepted for compatibility; the values come from the model file's header
    {"num-layers", 'N', 1, 'i'},
    {"hiddenstate-size", 'H', 1, 'i'},
    {"source-vocab-size", 'v', 1, 'i'},
    {"target-vocab-size", 'V', 1, 'i'},
    {"attention-model", 0, 1, 'i'},
    {"feed-input", 0, 1, 'i'},
    {"random-seed", 0, 1, 'i'},
    {"screen-print-rate", 0, 1, 'i'},
    {"print-beam", 0, 1, 'i'},
    // options of this program (no counterpart in the reference)
    {"attention-type", 0, 1, 'i'},  // local-p (default, what the reference's files hold) | global-dot
    {"dtype", 0, 1, 'i'},           // f32 (default) | bf16 | tf32 | f32-simt | f32-3xtf32 | f32-f16x2
    {"device-batch", 0, 1, 'i'},    // columns per device launch group (default 256 scoring, 32 sentences decoding)
    {"prep-only", 0, 0, 'i'},       // stop after writing the integer files into the tmp directory
    {"keep-tmp", 0, 0, 'i'},        // do not delete the tmp directory
    {"int-input", 0, 0, 'i'},       // the data files already hold integer records in the reference's tmp format
    // inference features outside this program
    {"multi-source", 0, 2, 'x'},
    {"decode-multi-source-data-files", 0, 2, 'x'},
    {"decode-multi-source-vocab-mappings", 0, 2, 'x'},
    {"char-mt", 0, 2, 'x'},
    {"stoch-gen", 'g', 2, 'x'},
    {"stoch-gen-len", 0, 1, 'x'},
    {"temperature", 0, 1, 'x'},
    {"fsa", 0, 1, 'x'},
    {"fsa-weight", 0, 1, 'x'},
    {"fsa-log", 0, 1, 'x'},
    {"interactive", 0, 1, 'x'},
    {"interactive-line", 0, 1, 'x'},
    {"repeat-penalty", 0, 1, 'x'},
    {"adjacent-repeat-penalty", 0, 1, 'x'},
    {"encourage-list", 0, 2, 'x'},
    {"encourage-weight", 0, 2, 'x'},
    {"wordlen-weight", 0, 1, 'x'},
    {"alliteration-weight", 0, 1, 'x'},
    {"lsh-type", 0, 1, 'x'},
    {"WTA-K", 0, 1, 'x'},
    {"WTA-units-per-band", 0, 1, 'x'},
    {"WTA-W", 0, 1, 'x'},
    {"WTA-m", 0, 1, 'x'},
    {"WTA-threshold", 0, 1, 'x'},
    {"WTA-topn", 0, 1, 'x'},
    {"target-vocab-policy", 0, 1, 'x'},
    {"top-vocab-size", 0, 1, 'x'},
    {"target-vocab-cap", 0, 1, 'x'},
    {"f2e-file", 0, 1, 'x'},
    {"pre-norm-ensemble", 0, 1, 'x'},
    {"NCE-score", 0, 1, 'x'},
    {"bi-directional", 0, 1, 'x'},
    // training
    {"train", 't', 2, 't'},
    {"cont-train", 'C', 2, 't'},
    {"vocab-mapping-file", 0, 1, 't'},
    {"dropout", 'd', 1, 't'},
    {"learning-rate", 'l', 1, 't'},
    {"parameter-range", 'P', 2, 't'},
    {"number-epochs", 'n', 1, 't'},
    {"matrix-clip-gradients", 'c', 1, 't'},
    {"whole-clip-gradients", 'w', 1, 't'},
    {"adaptive-halve-lr", 'a', 2, 't'},
    {"adaptive-decrease-factor", 'A', 1, 't'},
    {"fixed-halve-lr", 0, 1, 't'},
    {"fixed-halve-lr-full", 0, 1, 't'},
    {"best-model", 'B', 1, 't'},
    {"save-all-models", 0, 1, 't'},
    {"truncated-softmax", 'T', 2, 't'},
    {"NCE", 0, 1, 't'},
    {"shuffle", 0, 1, 't'},
    {"UNK-replacement", 0, 1, 't'},
    {"clip-cell", 0, 2, 't'},
};

struct Options {
  std::map<std::string, std::vector<std::string>> values;
  bool has(const std::string& k) const { return values.count(k) != 0; }
  const std::vector<std::string>& all(const std::string& k) const { return values.at(k); }
  std::string one(const std::string& k) const {
    const auto& v = values.at(k);
    if (v.size() != 1) die("option --" + k + " takes exactly one value");
    return v[0];
  }
};

const OptSpec* find_long(const std::string& n) {
  for (const auto& o : kOptions)
    if (n == o.name) return &o;
  return nullptr;
}
const OptSpec* find_short(char c) {
  for (const auto& o : kOptions)
    if (o.short_name && o.short_name == c) return &o;
  return nullptr;
}
bool looks_like_number(const std::string& s) {
  char* e;
  strtod(s.c_str(), &e);
  return !s.empty() && *e == 0;
}
// a token opens a new option when it is "--name", or "-x" for a declared short name (and is not a negative number)
const OptSpec* option_of(const std::string& tok, std::string* inline_value) {
  inline_value->clear();
  if (tok.size() > 2 && tok[0] == '-' && tok[1] == '-') {
    std::string n = tok.substr(2);
    const size_t eq = n.find('=');
    if (eq != std::string::npos) { *inline_value = n.substr(eq + 1); n = n.substr(0, eq); }
    const OptSpec* o = find_long(n);
    if (!o) die("unrecognised option '" + tok + "'");
    return o;
  }
  if (tok.size() >= 2 && tok[0] == '-' && tok[1] != '-' && !looks_like_number(tok)) {
    const OptSpec* o = find_short(tok[1]);
    if (!o) die("unrecognised option '" + tok + "'");
    if (tok.size() > 2) *inline_value = tok.substr(2);
    return o;
  }
  return nullptr;
}

Options parse_options(int argc, char** argv) {
  Options opt;
  int i = 1;
  while (i < argc) {
    std::string inl;
    const OptSpec* o = option_of(argv[i], &inl);
    if (!o) die(std::string("too many positional options: '") + argv[i] + "'");
    ++i;
    std::vector<std::string>& dst = opt.values[o->name];
    if (!inl.empty()) dst.push_back(inl);
    if (o->arity == 1 && inl.empty()) {
      if (i >= argc) die(std::string("the required argument for option '--") + o->name + "' is missing");
      dst.push_back(argv[i++]);
    } else if (o->arity == 2) {
      std::string dummy;
      while (i < argc && !option_of(argv[i], &dummy)) dst.push_back(argv[i++]);
      if (dst.empty()) die(std::string("the required argument for option '--") + o->name + "' is missing");
    }
  }
  return opt;
}

bool parse_bool(const std::string& s, const std::string& name) {
  if (s == "1" || s == "true" || s == "True" || s == "yes" || s == "on") return true;
  if (s == "0" || s == "false" || s == "False" || s == "no" || s == "off") return false;
  die("option --" + name + " wants a bool, got '" + s + "'");
}
int parse_int(const std::string& s, const std::string& name) {
  char* e;
  const long v = strtol(s.c_str(), &e, 10);
  if (s.empty() || *e) die("option --" + name + " wants an integer, got '" + s + "'");
  return (int)v;
}
double parse_double(const std::string& s, const std::string& name) {
  char* e;
  const double v = strtod(s.c_str(), &e);
  if (s.empty() || *e) die("option --" + name + " wants a number, got '" + s + "'");
  return v;
}

// ------------------------------------------------------------------------------------------------ parameters
// The subset of global_params (src/global_params.h) the inference paths read, with the reference's defaults.
struct Params {
  bool sequence = false;
  int minibatch = 8;       // -m
  int longest_sent = 100;  // -L
  int beam = 12;           // -b
  double penalty = 0;      // -p
  bool print_score = false;
  double min_ratio = 0.5, max_ratio = 1.5;  // --dec-ratio
  int attention_width = 10;
  bool legacy = false;
  std::string tmp_location = ".";
  std::string unique_dir;
  std::vector<int> gpus;
  int att_type = 0;  // 0: what the file says, as local-p
  int dtype = ZRNN_F32;
  int device_batch = 0;
  bool prep_only = false, keep_tmp = false, int_input = false;
  std::string unk_file;
};

void remove_tmp_dir(const Params& p) {
  if (p.unique_dir.empty() || p.keep_tmp) return;
  static const char* names[] = {"validation.txt", "decoder_output.txt"};
  for (const char* n : names) unlink((p.unique_dir + "/" + n).c_str());
  for (int k = 0; k < 8; ++k) unlink((p.unique_dir + "/kbest_tmp_" + std::to_string(k)).c_str());
  for (int k = 0; k < 64; ++k) unlink((p.unique_dir + "/part_" + std::to_string(k) + ".bin").c_str());
  rmdir(p.unique_dir.c_str());
}

// The reference creates <tmp-dir-location>/<random name>/ for its integer files and deletes it on exit
// (src/main.cu:270-300).
void make_tmp_dir(Params* p) {
  std::string templ = p->tmp_location + "/zoph_tmp_XXXXXX";
  std::vector<char> buf(templ.begin(), templ.end());
  buf.push_back(0);
  if (!mkdtemp(buf.data())) die("cannot create a tmp directory under " + p->tmp_location);
  p->unique_dir = buf.data();
  logger << "Temp directory being created named: " << p->unique_dir << "\n";
}

void check_status(int st, const char* what) {
  if (st != ZRNN_OK) die(std::string(what) + ": " + zrnn_status_string(st) + ": " + zrnn_last_error());
}

zrnn_model* load_model(const Params& p, const std::string& path) {
  const auto t0 = std::chrono::steady_clock::now();
  zrnn_model* m = nullptr;
  check_status(zrnn_model_load_file(path.c_str(), p.att_type, p.attention_width, p.dtype, &m), "loading the model");
  const double sec = std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
  zrnn_model_config c;
  zrnn_model_get_config(m, &c);
  logger << "Model loaded in " << sec << " seconds: layers " << c.num_layers << ", hiddenstate size " << c.H
         << ", target vocab " << c.V_tgt << ", source vocab " << c.V_src << ", attention " << c.attention
         << ", feed input " << c.feed_input << "\n";
  return m;
}

void select_device(const Params& p) {
  int n = 0;
  check_status(zrnn_device_count(&n), "querying devices");
  if (n <= 0) die("no CUDA device is visible; this program has no CPU path");
  for (int g : p.gpus)
    if (g < 0 || g >= n) die("--multi-gpu names device " + std::to_string(g) + " but only " + std::to_string(n) + " are visible");
  if (!p.gpus.empty()) check_status(zrnn_set_device(p.gpus[0]), "selecting the device");
}

// ------------------------------------------------------------------------------------------------ sentence sharding
// The reference's -M g0 g1 ... gsoftmax places the layers and the softmax on those devices (src/main.cu:154,
// src/model.hpp:34-51) and still runs one minibatch at a time.  Sentences are independent in the forward path, so
// here every DISTINCT device named by -M gets a worker process that holds the whole model and takes every W-th device
// batch; there is no exchange between the workers, and the parent merges their results in file order.  The workers
// are forked before the first CUDA call of the process (a CUDA runtime does not survive a fork) and hand their
// results back through files in the tmp directory.
std::vector<int> distinct_devices(const Params& p) {
  std::vector<int> d;
  for (int g : p.gpus)
    if (std::find(d.begin(), d.end(), g) == d.end()) d.push_back(g);
  return d;
}
struct Workers {
  int W = 1;    // worker processes
  int me = -1;  // -1: no sharding, this process does everything; >= 0: this process is worker `me`
  bool mine(int batch_index) const { return me < 0 || batch_index % W == me; }
};
std::string part_file(const Params& p, int w) { return p.unique_dir + "/part_" + std::to_string(w) + ".bin"; }
// Forks one worker per distinct device.  Returns in every worker (me >= 0, its device made the only one of p) and,
// after all workers have exited successfully, in the parent (me = -1, W = number of workers whose part files wait).
Workers fork_workers(Params* p, bool* is_parent_of_workers) {
  Workers wk;
  *is_parent_of_workers = false;
  const std::vector<int> dev = distinct_devices(*p);
  if (dev.size() < 2) return wk;
  wk.W = (int)dev.size();
  logger << "Sharding the sentences over " << wk.W << " devices:";
  for (int g : dev) logger << " " << g;
  logger << "\n";
  logger.flush();
  std::vector<pid_t> pids;
  for (int w = 0; w < wk.W; ++w) {
    const pid_t pid = fork();
    if (pid < 0) die("cannot fork a worker process");
    if (pid == 0) {
      wk.me = w;
      p->gpus.assign(1, dev[w]);
      return wk;
    }
    pids.push_back(pid);
  }
  bool ok = true;
  for (size_t w = 0; w < pids.size(); ++w) {
    int st = 0;
    if (waitpid(pids[w], &st, 0) < 0 || !WIFEXITED(st) || WEXITSTATUS(st) != 0) {
      logger << "ERROR: the worker on device " << dev[w] << " failed\n";
      ok = false;
    }
  }
  if (!ok) { remove_tmp_dir(*p); die("sentence sharding: a worker failed"); }
  *is_parent_of_workers = true;
  return wk;
}
[[noreturn]] void worker_done() {
  logger.flush();
  _exit(0);
}
template <class T>
void put_vec(std::ofstream& os, const std::vector<T>& v) {
  const long long n = (long long)v.size();
  os.write((const char*)&n, sizeof(n));
  if (n) os.write((const char*)v.data(), sizeof(T) * v.size());
}
template <class T>
bool get_vec(std::ifstream& is, std::vector<T>* v) {
  long long n = 0;
  if (!is.read((char*)&n, sizeof(n)) || n < 0) return false;
  v->resize((size_t)n);
  return n == 0 || (bool)is.read((char*)v->data(), sizeof(T) * v->size());
}

void print_prep_stats(const PrepStats& st, bool have_source, const char* what) {
  if (have_source) {
    logger << "----------------------------source " << what << " file info-----------------------------\n";
    logger << "Number of source word tokens: " << st.src_tokens << "\n";
    logger << "Number of source segment pairs (lines in training file): " << st.lines << "\n";
    logger << "Longest source segment (after removing long sentences for training): " << st.longest_src << "\n";
    logger << "-------------------------------------------------------------------------------\n\n";
  }
  if (std::strcmp(what, "kbest") != 0) {
    logger << "----------------------------target " << what << " file info-----------------------------\n";
    logger << "Number of target word tokens: " << st.tgt_tokens << "\n";
    logger << "Number of target segment pairs (lines in training file): " << st.lines << "\n";
    logger << "Longest target segment (after removing long sentences for training): " << st.longest_tgt << "\n";
  }
  logger << "Total word tokens thrown out due to sentence cutoff: " << st.thrown_tokens << "\n";
  logger << "-------------------------------------------------------------------------------\n\n";
}

// ------------------------------------------------------------------------------------------------ force-decode
// neuralMT_model::get_perplexity (src/model.hpp:2281-2355): one line per minibatch of the integer file with the sum
// of ln p over its target words, then the perplexity over the whole file.  The reference evaluates one minibatch per
// forward pass; columns are independent in the forward path, so several minibatches ride in one device batch here
// and their columns are summed back per minibatch.
int run_force_decode(const Options& opt, Params& p) {
  const std::vector<std::string>& f = opt.all("force-decode");
  std::string src_file, tgt_file, model_file, out_file;
  if (p.int_input) {
    // --int-input: <integer minibatch file> <model.nn> <output file>, records already grouped by --minibatch-size
    if (f.size() != 3) die("force-decode with --int-input takes three arguements: 1. integer minibatch file 2. neural network file name 3. output file name");
    tgt_file = f[0]; model_file = f[1]; out_file = f[2];
  } else if (p.sequence) {
    if (f.size() != 3)
      die("force-decode takes three arguements 1.input file name (input sentences)2. neural network file name 3.output file name");
    tgt_file = f[0]; model_file = f[1]; out_file = f[2];
  } else {
    if (f.size() != 4)
      die("force-decode takes four arguements: 1. source input file 2. target input file  3. neural network file name 4. output file name");
    src_file = f[0]; tgt_file = f[1]; model_file = f[2]; out_file = f[3];
    if (src_file == tgt_file) die("do not use the same file for source and target data");
    p.minibatch = 1;  // src/main.cu:1160,1169: sequence-to-sequence force-decode always runs with minibatch 1
  }
  Vocab vocab;
  std::string err;
  if (!vocab.load(model_file, &err)) die(err);
  if (vocab.header.n_header_ints != 9) die("the model file is not in the correct format for force-decode");
  if (vocab.header.lm != p.sequence)
    die(p.sequence ? "--sequence was given but the model file holds a sequence-to-sequence model"
                   : "the model file holds a sequence model; pass --sequence");
  make_tmp_dir(&p);
  const std::string int_file = p.unique_dir + "/validation.txt";
  std::vector<Record> recs;
  PrepStats st;
  if (p.int_input) {
    if (!zrnn::text::read_minibatch_file(tgt_file, &recs, &err)) die(err);
  } else {
    const bool ok = p.sequence ? zrnn::text::prep_force_decode_lm(vocab, tgt_file, p.longest_sent, p.minibatch, &recs, &st, &err)
                               : zrnn::text::prep_force_decode_nonlm(vocab, src_file, tgt_file, p.longest_sent, p.minibatch, &recs, &st, &err);
    if (!ok) { remove_tmp_dir(p); die(err); }
    print_prep_stats(st, !p.sequence, "dev");
    if (!zrnn::text::write_minibatch_file(int_file, recs, &err)) die(err);
  }
  if (p.prep_only) {
    logger << "Integer minibatch file: " << int_file << "\n";
    return 0;
  }
  // units = the reference's minibatches; order them by length so a device batch carries little padding
  const int n_units = (int)((recs.size() + p.minibatch - 1) / p.minibatch);
  std::vector<int> unit_len(n_units, 0), order(n_units);
  for (int u = 0; u < n_units; ++u)
    for (int r = u * p.minibatch; r < std::min((int)recs.size(), (u + 1) * p.minibatch); ++r)
      unit_len[u] = std::max(unit_len[u], (int)(recs[r].tgt_in.size() + recs[r].src.size()));
  std::iota(order.begin(), order.end(), 0);
  std::stable_sort(order.begin(), order.end(), [&](int a, int b) { return unit_len[a] > unit_len[b]; });
  const int cap = p.device_batch > 0 ? p.device_batch : 256;
  std::vector<double> unit_sum(n_units, 0.0);
  long long total_target_words = 0;
  const auto t0 = std::chrono::steady_clock::now();
  bool merge = false;
  const Workers wk = fork_workers(&p, &merge);
  if (merge) {
    for (int w = 0; w < wk.W; ++w) {
      std::ifstream is(part_file(p, w).c_str(), std::ios::binary);
      std::vector<long long> words;
      std::vector<int> units;
      std::vector<double> sums;
      if (!is || !get_vec(is, &words) || !get_vec(is, &units) || !get_vec(is, &sums) || words.size() != 1 ||
          units.size() != sums.size())
        die("sentence sharding: cannot read " + part_file(p, w));
      total_target_words += words[0];
      for (size_t i = 0; i < units.size(); ++i) unit_sum[units[i]] += sums[i];
    }
  } else {
    select_device(p);
    zrnn_model* model = load_model(p, model_file);
    std::vector<float> logp;
    std::vector<int> my_units;
    int batch_index = 0;
    for (int u0 = 0; u0 < n_units; ++batch_index) {
      std::vector<int> rows;
      int u1 = u0;
      const int first = u1;
      while (u1 < n_units && (rows.empty() || (int)rows.size() + p.minibatch <= cap)) {
        const int u = order[u1++];
        for (int r = u * p.minibatch; r < std::min((int)recs.size(), (u + 1) * p.minibatch); ++r) rows.push_back(r);
      }
      u0 = u1;
      if (!wk.mine(batch_index)) continue;
      for (int i = first; i < u1; ++i) my_units.push_back(order[i]);
      const Minibatch mb = zrnn::text::make_minibatch(recs, rows);
      total_target_words += mb.target_words;
      logp.assign((size_t)mb.T * mb.B, 0.f);
      double total = 0;
      check_status(zrnn_score_batch(model, p.sequence ? nullptr : mb.src.data(), mb.S_max, mb.tgt_in.data(),
                                    mb.tgt_out.data(), mb.T, mb.B, logp.data(), &total), "scoring");
      for (int b = 0; b < mb.B; ++b) {
        double s = 0;
        for (int t = 0; t < mb.T; ++t) s += logp[(size_t)b + (size_t)t * mb.B];
        unit_sum[rows[b] / p.minibatch] += s;
      }
    }
    zrnn_model_destroy(model);
    if (wk.me >= 0) {
      std::ofstream os(part_file(p, wk.me).c_str(), std::ios::binary);
      std::vector<double> sums;
      for (int u : my_units) sums.push_back(unit_sum[u]);
      put_vec(os, std::vector<long long>(1, total_target_words));
      put_vec(os, my_units);
      put_vec(os, sums);
      os.close();
      if (!os) die("sentence sharding: cannot write " + part_file(p, wk.me));
      worker_done();
    }
  }
  const double sec = std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
  std::ofstream fd(out_file.c_str());
  if (!fd) die("cannot write " + out_file);
  double p_data = 0;
  for (int u = 0; u < n_units; ++u) {
    fd << unit_sum[u] << "\n";  // default stream formatting, as the reference's fd_stream << temp
    p_data += unit_sum[u];
  }
  fd.close();
  p_data /= std::log(2.0);
  const double perplexity = std::pow(2.0, -p_data / (double)total_target_words);
  logger << "Total target words: " << total_target_words << "\n";
  logger << std::setprecision(15) << "Perplexity dev set: " << perplexity << "\n";
  logger << std::setprecision(15) << "P_data dev set: " << p_data << "\n";
  logger << std::setprecision(6) << "Scored " << (int)recs.size() << " sentences in " << sec << " seconds ("
         << (double)total_target_words / sec << " target words per second)\n";
  return 0;
}

// ------------------------------------------------------------------------------------------------ decode
// ensemble_factory::decode_file (src/ensemble_factory.hpp:583-765) + decoder::output_k_best_hypotheses
// (src/decoder.h:1386-1463): for every kept source line a line of dashes, then up to k hypotheses (each optionally
// preceded by "-Score: x") as rows of target ids each followed by a blank, then an empty line; unint_file turns the
// id rows into words (src/main.cu:1613).
int run_decode(const Options& opt, Params& p) {
  const std::vector<std::string>& k = opt.all("decode");
  if (k.size() < 3) die("at least 3 arguements must be entered for --decode, 1. number of best outputs 2. neural network file name (this is the output file you get after training the neural network) 3. output file name");
  if (!opt.has("decode-main-data-files")) die("--decode needs --decode-main-data-files <data file 1> ...");
  const std::vector<std::string>& data_files = opt.all("decode-main-data-files");
  const int num_hypotheses = parse_int(k[0], "decode");
  std::vector<std::string> model_names(k.begin() + 1, k.end() - 1);
  const std::string final_file = k.back();
  if (model_names.size() != data_files.size()) die("the same number of inputs must be specified as models");
  const int K = (int)model_names.size();
  if (K > 8) die("at most 8 models can be ensembled");
  if (p.beam <= 0) die("beam size cannot be <=0");
  if (p.penalty < 0) die("penalty cannot be less than zero");
  if (num_hypotheses <= 0) die("the number of outputs must be positive");
  if (p.min_ratio >= p.max_ratio) die("min decoding ratio must be <= max_decoding_ratio");

  // every model of an ensemble has its own source vocabulary and data file; they share the target vocabulary, and
  // the first model's mapping turns the output back into words (src/main.cu:1038-1046, 1611-1613)
  std::vector<Vocab> vocabs(K);
  std::string err;
  for (int k = 0; k < K; ++k) {
    if (!vocabs[k].load(model_names[k], &err)) die(err);
    if (vocabs[k].header.lm) die("--decode needs a sequence-to-sequence model");
    if (vocabs[k].header.V_tgt != vocabs[0].header.V_tgt) die("ensembled models must share the target vocabulary");
  }
  const Vocab& vocab = vocabs[0];
  make_tmp_dir(&p);
  const std::string int_out = p.unique_dir + "/decoder_output.txt";
  std::vector<std::vector<std::vector<int>>> sents_k(K);
  for (int k = 0; k < K; ++k) {
    const std::string int_file = p.unique_dir + "/kbest_tmp_" + std::to_string(k);
    std::vector<int> kept;
    PrepStats st;
    if (p.int_input) {
      if (!zrnn::text::read_kbest_file(data_files[k], &sents_k[k], &err)) die(err);
    } else {
      if (!zrnn::text::prep_kbest(vocabs[k], data_files[k], p.longest_sent, p.legacy, &sents_k[k], &kept, &st, &err)) die(err);
      print_prep_stats(st, true, "kbest");
      if (!zrnn::text::write_kbest_file(int_file, sents_k[k], &err)) die(err);
    }
    if (p.prep_only) logger << "Integer decode file: " << int_file << "\n";
    // the reference walks the K integer files in lock step; files that kept different lines would pair up the wrong
    // sentences, so that case is an error here
    if (sents_k[k].size() != sents_k[0].size())
      die("data file " + std::to_string(k) + " keeps " + std::to_string(sents_k[k].size()) + " sentences after the length cut-off, data file 0 keeps " + std::to_string(sents_k[0].size()));
  }
  if (p.prep_only) return 0;
  const std::vector<std::vector<int>>& sents = sents_k[0];
  const int n = (int)sents.size();
  const int Lmax = p.longest_sent + 4;
  std::vector<int> all_len((size_t)n * num_hypotheses, 0);
  std::vector<float> all_score((size_t)n * num_hypotheses, 0.f);
  std::vector<int> all_ids((size_t)n * num_hypotheses * Lmax, -1);
  const bool unk = !p.unk_file.empty();  // --UNK-decode: BZ_CUDA::unk_replacement (src/main.cu:410-412)
  std::vector<int> all_align(unk ? (size_t)n * num_hypotheses * Lmax : 0, -1);
  // decode the sentences in groups of similar length; results go back to file order
  std::vector<int> order(n);
  std::iota(order.begin(), order.end(), 0);
  std::stable_sort(order.begin(), order.end(), [&](int a, int b) { return sents[a].size() > sents[b].size(); });
  const int group = p.device_batch > 0 ? p.device_batch : 32;
  const auto t0 = std::chrono::steady_clock::now();
  long long out_words = 0;
  bool merge = false;
  const Workers wk = fork_workers(&p, &merge);
  // copies the hypotheses of sentence `s` from a group's arrays (position i) into the file-order arrays
  auto keep = [&](int s, size_t i, const std::vector<int>& ids, const std::vector<int>& len, const std::vector<float>& score,
                  const std::vector<int>& align) {
    const size_t dst = (size_t)s * num_hypotheses;
    for (int h = 0; h < num_hypotheses; ++h) {
      all_len[dst + h] = len[i * num_hypotheses + h];
      all_score[dst + h] = score[i * num_hypotheses + h];
      std::memcpy(&all_ids[(dst + h) * Lmax], &ids[(i * num_hypotheses + h) * Lmax], sizeof(int) * Lmax);
      if (unk) std::memcpy(&all_align[(dst + h) * Lmax], &align[(i * num_hypotheses + h) * Lmax], sizeof(int) * Lmax);
      out_words += all_len[dst + h];
    }
  };
  if (merge) {
    for (int w = 0; w < wk.W; ++w) {
      std::ifstream is(part_file(p, w).c_str(), std::ios::binary);
      std::vector<int> which, ids, len, align;
      std::vector<float> score;
      if (!is || !get_vec(is, &which) || !get_vec(is, &ids) || !get_vec(is, &len) || !get_vec(is, &score) ||
          !get_vec(is, &align) || len.size() != which.size() * (size_t)num_hypotheses || score.size() != len.size() ||
          ids.size() != len.size() * (size_t)Lmax || (unk && align.size() != ids.size()))
        die("sentence sharding: cannot read " + part_file(p, w));
      for (size_t i = 0; i < which.size(); ++i) keep(which[i], i, ids, len, score, align);
    }
  } else {
    select_device(p);
    std::vector<zrnn_model*> models(K);
    for (int k = 0; k < K; ++k) models[k] = load_model(p, model_names[k]);
    zrnn_model* model = models[0];
    zrnn_model_config cfg;
    zrnn_model_get_config(model, &cfg);
    const int cap_beam = (int)std::floor(std::sqrt((double)cfg.V_tgt));
    if (p.beam > cap_beam) logger << "Note: beam size " << p.beam << " is capped at floor(sqrt(target vocab)) = " << cap_beam << "\n";
    std::vector<int> my_which, my_ids, my_len, my_align;
    std::vector<float> my_score;
    for (int g0 = 0, batch_index = 0; g0 < n; g0 += group, ++batch_index) {
      if (!wk.mine(batch_index)) continue;
      const int g1 = std::min(n, g0 + group), ng = g1 - g0;
      std::vector<std::vector<int>> flat_k(K), lens_k(K);
      for (int k = 0; k < K; ++k)
        for (int i = g0; i < g1; ++i) {
          const auto& s = sents_k[k][order[i]];
          if (s.empty()) die("source line with no words cannot be decoded");
          flat_k[k].insert(flat_k[k].end(), s.begin(), s.end());
          lens_k[k].push_back((int)s.size());
        }
      const std::vector<int>&flat = flat_k[0], &lens = lens_k[0];
      std::vector<int> ids((size_t)ng * num_hypotheses * Lmax), len((size_t)ng * num_hypotheses);
      std::vector<float> score((size_t)ng * num_hypotheses);
      std::vector<int> align(unk ? ids.size() : 0);
      if (K == 1) {
        check_status(zrnn_beam_decode_batch_align(model, flat.data(), lens.data(), ng, p.beam, num_hypotheses,
                                                  (float)p.min_ratio, (float)p.max_ratio, (float)p.penalty, p.longest_sent,
                                                  ids.data(), len.data(), score.data(), unk ? align.data() : nullptr),
                     "decoding");
      } else {
        std::vector<const int*> fp(K), lp(K);
        for (int k = 0; k < K; ++k) { fp[k] = flat_k[k].data(); lp[k] = lens_k[k].data(); }
        check_status(zrnn_beam_decode_ensemble_align(models.data(), K, fp.data(), lp.data(), ng, p.beam, num_hypotheses,
                                                     (float)p.min_ratio, (float)p.max_ratio, (float)p.penalty,
                                                     p.longest_sent, ids.data(), len.data(), score.data(),
                                                     unk ? align.data() : nullptr), "ensemble decoding");
      }
      for (int i = 0; i < ng; ++i) keep(order[g0 + i], (size_t)i, ids, len, score, align);
      if (wk.me >= 0) {
        for (int i = 0; i < ng; ++i) my_which.push_back(order[g0 + i]);
        my_ids.insert(my_ids.end(), ids.begin(), ids.end());
        my_len.insert(my_len.end(), len.begin(), len.end());
        my_score.insert(my_score.end(), score.begin(), score.end());
        my_align.insert(my_align.end(), align.begin(), align.end());
      }
      logger << "Decoded " << g1 << " of " << n << " sentences" << (wk.me >= 0 ? " (device " + std::to_string(p.gpus[0]) + ")" : "") << "\n";
    }
    for (zrnn_model* m : models) zrnn_model_destroy(m);
    if (wk.me >= 0) {
      std::ofstream os(part_file(p, wk.me).c_str(), std::ios::binary);
      put_vec(os, my_which);
      put_vec(os, my_ids);
      put_vec(os, my_len);
      put_vec(os, my_score);
      put_vec(os, my_align);
      os.close();
      if (!os) die("sentence sharding: cannot write " + part_file(p, wk.me));
      worker_done();
    }
  }
  const double sec = std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
  {
    std::ofstream os(int_out.c_str());
    if (!os) die("cannot write " + int_out);
    std::ofstream unk_os;
    if (unk) {
      unk_os.open(p.unk_file.c_str());
      if (!unk_os) die("cannot write " + p.unk_file);
    }
    for (int s = 0; s < n; ++s) {
      os << "------------------------------------------------\n";
      for (int h = 0; h < num_hypotheses; ++h) {
        const size_t at = (size_t)s * num_hypotheses + h;
        if (all_len[at] <= 0) continue;
        if (p.print_score) os << "-Score: " << all_score[at] << "\n";
        for (int j = 0; j < all_len[at]; ++j) os << all_ids[at * Lmax + j] << " ";
        os << "\n";
        if (unk) {
          // one line per hypothesis: for every <UNK> (id 2) at position j the alignment stored at j + 1
          // (src/decoder.h:1452-1459)
          for (int j = 0; j < all_len[at]; ++j)
            if (all_ids[at * Lmax + j] == 2 && j + 1 < Lmax) unk_os << all_align[at * Lmax + j + 1] << " ";
          unk_os << "\n";
        }
      }
      os << "\n";
    }
  }
  if (!zrnn::text::unint_file(vocab, int_out, final_file, true, &err)) die(err);
  logger << std::setprecision(6) << "Decoded " << n << " sentences in " << sec << " seconds (" << (double)out_words / sec
         << " output words per second)\n";
  return 0;
}

void print_help() {
  std::cout <<
      "B200 inference front end for Zoph_RNN models.\n"
      "  -f, --force-decode <source file> <target file> <model.nn> <output file>\n"
      "        with -s: <target file> <model.nn> <output file>; one sum of ln p per minibatch, perplexity to the log\n"
      "  -k, --decode <how many outputs> <model.nn> [<model.nn> ...] <output file>\n"
      "        with --decode-main-data-files <source file> [<source file> ...], one per model (ensemble decoding)\n"
      "  -s, --sequence          the model is a sequence (language) model\n"
      "  -b, --beam-size N       beam size for --decode (default 12)\n"
      "  -p, --penalty X         word penalty added per target word for --decode (default 0)\n"
      "      --print-score B     print the unnormalised log-probability of every hypothesis\n"
      "      --dec-ratio MIN MAX decoding length ratios (default 0.5 1.5)\n"
      "  -L, --longest-sent N    maximum sentence length (default 100)\n"
      "  -m, --minibatch-size N  minibatch size of the sequence force-decode (default 8)\n"
      "  -M, --multi-gpu I ...   device indices; every distinct device gets a worker process with the whole model and\n"
      "                          a share of the sentences (the reference places layers on them instead)\n"
      "      --attention-width D local attention half window (default 10)\n"
      "      --tmp-dir-location DIR, --logfile FILE, --legacy-model B\n"
      "  options of this program: --attention-type local-p|global-dot, --dtype f32|bf16|tf32|f32-simt|f32-3xtf32|f32-f16x2,\n"
      "      --device-batch N, --prep-only, --keep-tmp, --int-input\n";
}

}  // namespace

int main(int argc, char** argv) {
  Options opt = parse_options(argc, argv);
  if (opt.has("help") || argc == 1) {
    print_help();
    return 0;
  }
  if (opt.has("logfile")) logger.file.open(opt.one("logfile").c_str());
  for (const auto& kv : opt.values) {
    const OptSpec* o = find_long(kv.first);
    if (o->scope == 't') die("--" + kv.first + " belongs to training, which this program does not do (inference only: --force-decode, --decode)");
    if (o->scope == 'x') die("--" + kv.first + " selects a feature that is outside this program (single-source word models, no FSA / LSH / vocabulary shrinking)");
  }
  Params p;
  p.sequence = opt.has("sequence");
  if (opt.has("minibatch-size")) p.minibatch = parse_int(opt.one("minibatch-size"), "minibatch-size");
  if (opt.has("longest-sent")) p.longest_sent = parse_int(opt.one("longest-sent"), "longest-sent");
  if (opt.has("beam-size")) p.beam = parse_int(opt.one("beam-size"), "beam-size");
  if (opt.has("penalty")) p.penalty = parse_double(opt.one("penalty"), "penalty");
  if (opt.has("print-score")) p.print_score = parse_bool(opt.one("print-score"), "print-score");
  if (opt.has("legacy-model")) p.legacy = parse_bool(opt.one("legacy-model"), "legacy-model");
  if (opt.has("attention-width")) p.attention_width = parse_int(opt.one("attention-width"), "attention-width");
  if (opt.has("tmp-dir-location")) p.tmp_location = opt.one("tmp-dir-location");
  if (opt.has("device-batch")) p.device_batch = parse_int(opt.one("device-batch"), "device-batch");
  if (opt.has("UNK-decode")) p.unk_file = opt.one("UNK-decode");
  p.prep_only = opt.has("prep-only");
  p.keep_tmp = opt.has("keep-tmp") || p.prep_only;
  p.int_input = opt.has("int-input");
  if (opt.has("dec-ratio")) {
    const auto& r = opt.all("dec-ratio");
    if (r.size() != 2) die("only two inputs for decoding ratio");
    p.min_ratio = parse_double(r[0], "dec-ratio");
    p.max_ratio = parse_double(r[1], "dec-ratio");
  }
  if (opt.has("multi-gpu"))
    for (const auto& s : opt.all("multi-gpu")) p.gpus.push_back(parse_int(s, "multi-gpu"));
  if (opt.has("attention-type")) {
    const std::string t = opt.one("attention-type");
    if (t == "local-p") p.att_type = ZRNN_ATT_LOCAL_P;
    else if (t == "global-dot") p.att_type = ZRNN_ATT_GLOBAL_DOT;
    else die("--attention-type is local-p or global-dot");
  }
  if (opt.has("dtype")) {
    const std::string t = opt.one("dtype");
    if (t == "f32") p.dtype = ZRNN_F32;
    else if (t == "bf16") p.dtype = ZRNN_BF16;
    else if (t == "tf32") p.dtype = ZRNN_TF32;
    else if (t == "f32-simt") p.dtype = ZRNN_F32_SIMT;
    else if (t == "f32-3xtf32") p.dtype = ZRNN_F32_3XTF32;
    else if (t == "f32-f16x2") p.dtype = ZRNN_F32_F16X2;
    else die("--dtype is f32, bf16, tf32, f32-simt, f32-3xtf32 or f32-f16x2");
  }
  if (p.minibatch <= 0) die("minibatch size must be positive");
  if (p.longest_sent < 4) die("longest-sent is too small");
  int rc = 0;
  if (opt.has("decode")) rc = run_decode(opt, p);
  else if (opt.has("force-decode")) rc = run_force_decode(opt, p);
  else die("nothing to do: give --force-decode or --decode (training is outside this program)");
  remove_tmp_dir(p);
  logger.flush();
  return rc;
}
