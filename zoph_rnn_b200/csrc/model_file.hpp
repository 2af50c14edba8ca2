// Reader for the reference's text weight file ("model.nn").
// Format (src/model.hpp:2015-2088 writer, :2172-2241 reader, src/Eigen_Util.h:83-112 matrix reader):
//   line 1: integers  num_layers LSTM_size target_vocab source_vocab attention feed_input multi_source
//           combine_LSTM char_cnn   (src/add_model_info.h:7-9; older files carry only the first four)
//   line 2: a line of '=' ; source vocabulary lines "id word" ; '=' line   (absent for sequence models)
//   target vocabulary lines ; '=' line
//   then every matrix: `rows` lines of `cols` space-separated decimals followed by one empty line,
//   in the order given by the model's tensor list.
#pragma once
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>

namespace zrnn {

struct ModelFileHeader {
  int num_layers = 0, H = 0, V_tgt = 0, V_src = 0, attention = 0, feed_input = 0, multi_source = 0, combine = 0,
      char_cnn = 0;
  bool lm = false;
};

class ModelFileReader {
 public:
  ~ModelFileReader() { if (f_) fclose(f_); }
  // Opens the file, parses the header and skips the vocabulary mappings.
  bool open(const std::string& path, ModelFileHeader* h, std::string* err) {
    f_ = fopen(path.c_str(), "rb");
    if (!f_) { *err = "cannot open " + path; return false; }
    std::string line;
    if (!getline(&line)) { *err = "empty model file"; return false; }
    int v[9] = {0, 0, 0, 0, 0, 0, 0, 0, 0};
    int n = 0;
    const char* p = line.c_str();
    while (n < 9) {
      char* e;
      long x = strtol(p, &e, 10);
      if (e == p) break;
      v[n++] = (int)x;
      p = e;
    }
    if (n < 4) { *err = "model file header needs at least 4 integers"; return false; }
    h->num_layers = v[0]; h->H = v[1]; h->V_tgt = v[2]; h->V_src = v[3];
    h->attention = v[4]; h->feed_input = v[5]; h->multi_source = v[6]; h->combine = v[7]; h->char_cnn = v[8];
    h->lm = (h->V_src <= 0);
    if (!getline(&line) || line.compare(0, 3, "===") != 0) { *err = "missing separator after header"; return false; }
    const int sections = h->lm ? 1 : 2;
    for (int s = 0; s < sections; ++s) {
      bool found = false;
      while (getline(&line))
        if (line.compare(0, 3, "===") == 0) { found = true; break; }
      if (!found) { *err = "truncated vocabulary section"; return false; }
    }
    return true;
  }
  // Reads one rows x cols matrix into column-major storage.
  bool read_matrix(int rows, int cols, float* out, std::string* err) {
    std::string line;
    for (int r = 0; r < rows; ++r) {
      if (!getline(&line)) { *err = "truncated matrix (file ended)"; return false; }
      const char* p = line.c_str();
      for (int c = 0; c < cols; ++c) {
        char* e;
        const float x = strtof(p, &e);
        if (e == p) { *err = "truncated matrix row (expected " + std::to_string(cols) + " values)"; return false; }
        out[(size_t)c * rows + r] = x;
        p = e;
      }
    }
    getline(&line);  // the blank line that ends every matrix
    return true;
  }

 private:
  bool getline(std::string* s) {
    s->clear();
    if (!f_) return false;
    char buf[1 << 16];
    bool any = false;
    while (fgets(buf, sizeof(buf), f_)) {
      any = true;
      const size_t n = strlen(buf);
      s->append(buf, n);
      if (n && buf[n - 1] == '\n') { s->pop_back(); break; }
    }
    return any;
  }
  FILE* f_ = nullptr;
};

}  // namespace zrnn
