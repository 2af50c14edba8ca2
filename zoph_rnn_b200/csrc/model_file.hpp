// Reader for the reference's text weight file ("model.nn").
// Format (src/model.hpp:2015-2088 writer, :2172-2241 reader, src/Eigen_Util.h:83-112 matrix reader):
//   line 1: integers  num_layers LSTM_size target_vocab source_vocab attention feed_input multi_source
//           combine_LSTM char_cnn   (src/add_model_info.h:7-9; older files carry only the first four)
//   line 2: a line of '=' ; source vocabulary lines "id word" ; '=' line   (absent for sequence models)
//   target vocabulary lines ; '=' line
//   then every matrix: `rows` lines of `cols` space-separated decimals followed by one empty line,
//   in the order given by the model's tensor list.
//
// The reference parses the file with one istringstream per line, which takes minutes at V = 50k, H = 1000
// (two 50M-value matrices, about 1.2 GB of text).  Here the file is memory-mapped, line starts are found with
// memchr and the rows of a matrix are converted by a pool of threads with std::from_chars (correctly rounded,
// like the stream extraction it replaces), so start-up is bounded by page-cache bandwidth.
#pragma once
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <atomic>
#include <charconv>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <thread>
#include <utility>
#include <vector>

namespace zrnn {

struct ModelFileHeader {
  int num_layers = 0, H = 0, V_tgt = 0, V_src = 0, attention = 0, feed_input = 0, multi_source = 0, combine = 0,
      char_cnn = 0;
  int n_header_ints = 0;  // how many integers line 1 carried (the reference's -f path insists on 9)
  bool lm = false;
};

typedef std::vector<std::pair<int, std::string>> VocabList;  // (id, word) in file order

class ModelFileReader {
 public:
  ~ModelFileReader() { close(); }
  void close() {
    if (base_ && base_ != (const char*)MAP_FAILED && size_) munmap((void*)base_, size_);
    base_ = nullptr;
    size_ = 0;
    if (fd_ >= 0) ::close(fd_);
    fd_ = -1;
  }
  // Opens the file, parses the header and the vocabulary mappings; the cursor is left on the first matrix.
  bool open(const std::string& path, ModelFileHeader* h, std::string* err) {
    close();
    fd_ = ::open(path.c_str(), O_RDONLY);
    if (fd_ < 0) { *err = "cannot open " + path; return false; }
    struct stat sb;
    if (fstat(fd_, &sb) != 0 || sb.st_size <= 0) { *err = "empty model file"; return false; }
    size_ = (size_t)sb.st_size;
    base_ = (const char*)mmap(nullptr, size_, PROT_READ, MAP_PRIVATE, fd_, 0);
    if (base_ == (const char*)MAP_FAILED) { base_ = nullptr; *err = "cannot map " + path; return false; }
    madvise((void*)base_, size_, MADV_SEQUENTIAL);
    cur_ = 0;
    const char *b, *e;
    if (!next_line(&b, &e)) { *err = "empty model file"; return false; }
    int v[9] = {0, 0, 0, 0, 0, 0, 0, 0, 0};
    int n = 0;
    {
      std::string line(b, e);
      const char* p = line.c_str();
      while (n < 9) {
        char* q;
        long x = strtol(p, &q, 10);
        if (q == p) break;
        v[n++] = (int)x;
        p = q;
      }
    }
    if (n < 4) { *err = "model file header needs at least 4 integers"; return false; }
    h->n_header_ints = n;
    h->num_layers = v[0]; h->H = v[1]; h->V_tgt = v[2]; h->V_src = v[3];
    h->attention = v[4]; h->feed_input = v[5]; h->multi_source = v[6]; h->combine = v[7]; h->char_cnn = v[8];
    h->lm = (h->V_src <= 0);
    if (!next_line(&b, &e) || !is_separator(b, e)) { *err = "missing separator after header"; return false; }
    src_vocab_.clear();
    tgt_vocab_.clear();
    const int sections = h->lm ? 1 : 2;
    for (int s = 0; s < sections; ++s) {
      VocabList& dst = (s == 0 && !h->lm) ? src_vocab_ : tgt_vocab_;
      bool found = false;
      while (next_line(&b, &e)) {
        if (is_separator(b, e)) { found = true; break; }
        // "id word": the id, blanks, then the word up to the next blank (src/input_file_prep.h:2006-2010)
        const char* p = b;
        while (p < e && (*p == ' ' || *p == '\t')) ++p;
        int id = 0;
        auto r = std::from_chars(p, e, id);
        if (r.ec != std::errc()) continue;
        p = r.ptr;
        while (p < e && (*p == ' ' || *p == '\t')) ++p;
        const char* w = p;
        while (p < e && *p != ' ' && *p != '\t' && *p != '\r') ++p;
        // a mapping to an id outside the model's vocabulary would later index past the embedding table
        const int vsize = (s == 0 && !h->lm) ? h->V_src : h->V_tgt;
        if (id < 0 || id >= vsize) {
          *err = "vocabulary line maps '" + std::string(w, p) + "' to id " + std::to_string(id) + ", outside the model's " +
                 std::to_string(vsize) + " words";
          return false;
        }
        dst.emplace_back(id, std::string(w, p));
      }
      if (!found) { *err = "truncated vocabulary section"; return false; }
    }
    return true;
  }
  const VocabList& source_vocab() const { return src_vocab_; }
  const VocabList& target_vocab() const { return tgt_vocab_; }

  // Reads one rows x cols matrix into column-major storage (out[c * rows + r]).
  bool read_matrix(int rows, int cols, float* out, std::string* err) {
    std::vector<const char*> lb((size_t)rows), le((size_t)rows);
    for (int r = 0; r < rows; ++r)
      if (!next_line(&lb[r], &le[r])) { *err = "truncated matrix (file ended)"; return false; }
    {
      const char *b, *e;
      next_line(&b, &e);  // the blank line that ends every matrix
    }
    int nt = 1;
    if ((size_t)rows * cols >= (size_t)1 << 16) {
      nt = (int)std::thread::hardware_concurrency();
      if (const char* s = getenv("ZRNN_LOAD_THREADS")) nt = atoi(s);
      if (nt > 32) nt = 32;
      if (nt > rows) nt = rows;
      if (nt < 1) nt = 1;
    }
    std::atomic<int> bad_row(-1);
    auto work = [&](int r0, int r1) {
      for (int r = r0; r < r1 && bad_row.load(std::memory_order_relaxed) < 0; ++r)
        if (!parse_row(lb[r], le[r], cols, out + r, (size_t)rows)) bad_row.store(r);
    };
    if (nt == 1) {
      work(0, rows);
    } else {
      std::vector<std::thread> pool;
      const int per = (rows + nt - 1) / nt;
      for (int t = 0; t < nt; ++t) {
        const int r0 = t * per, r1 = r0 + per < rows ? r0 + per : rows;
        if (r0 < r1) pool.emplace_back(work, r0, r1);
      }
      for (auto& th : pool) th.join();
    }
    if (bad_row.load() >= 0) {
      *err = "truncated matrix row " + std::to_string(bad_row.load()) + " (expected " + std::to_string(cols) + " values)";
      return false;
    }
    return true;
  }

 private:
  static bool is_separator(const char* b, const char* e) { return e - b >= 3 && b[0] == '=' && b[1] == '=' && b[2] == '='; }
  bool next_line(const char** b, const char** e) {
    if (!base_ || cur_ >= size_) return false;
    const char* p = base_ + cur_;
    const char* nl = (const char*)memchr(p, '\n', size_ - cur_);
    *b = p;
    *e = nl ? nl : base_ + size_;
    cur_ = nl ? (size_t)(nl - base_) + 1 : size_;
    return true;
  }
  // cols decimals separated by blanks; value c goes to out[c * stride]
  static bool parse_row(const char* p, const char* e, int cols, float* out, size_t stride) {
    for (int c = 0; c < cols; ++c) {
      while (p < e && (*p == ' ' || *p == '\t' || *p == '\r')) ++p;
      if (p >= e) return false;
      float x;
      auto r = std::from_chars(p, e, x);
      if (r.ec == std::errc()) {
        p = r.ptr;
      } else {
        // forms from_chars refuses (leading '+', out-of-range magnitudes that strtof saturates): same result as strtof
        const char* q = p;
        while (q < e && *q != ' ' && *q != '\t' && *q != '\r') ++q;
        std::string tok(p, q);
        char* end;
        x = strtof(tok.c_str(), &end);
        if (end == tok.c_str()) return false;
        p = q;
      }
      out[(size_t)c * stride] = x;
    }
    return true;
  }

  int fd_ = -1;
  const char* base_ = nullptr;
  size_t size_ = 0, cur_ = 0;
  VocabList src_vocab_, tgt_vocab_;
};

}  // namespace zrnn
