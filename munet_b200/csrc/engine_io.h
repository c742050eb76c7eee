// Host-side parsing for the executor: a small JSON reader and the loader for
// MuNet deploy artifacts (an uncompressed .npz = zip of .npy members holding a
// JSON module tree, named tensors and manifest metadata;
// src/inference_serialization.cpp:919-1033, documentation/guides/serialization.md).
#pragma once
#include <map>
#include <string>
#include <utility>
#include <vector>

namespace mu {

struct Json {
  enum Kind { NUL, BOOL, NUM, STR, ARR, OBJ } kind = NUL;
  bool b = false;
  double num = 0;
  std::string str;
  std::vector<Json> arr;
  std::vector<std::pair<std::string, Json>> obj;
  bool is_object() const { return kind == OBJ; }
  bool is_array() const { return kind == ARR; }
  bool is_string() const { return kind == STR; }
  bool is_number() const { return kind == NUM; }
  const Json *get(const char *key) const {
    for (auto &kv : obj)
      if (kv.first == key)
        return &kv.second;
    return nullptr;
  }
};

bool parse_json(const std::string &text, Json *out, std::string *why);

struct NamedTensor {
  int dtype = 0; // MuNet DataType order: 0 f32, 1 f16, 2 bf16, 3 i32
  std::vector<long long> shape;
  const void *data = nullptr;
  bool on_device = false;
  std::vector<unsigned char> owned; // backing store when loaded from a file
  long long numel() const {
    long long n = 1;
    for (long long s : shape)
      n *= s;
    return n;
  }
};

// Parses and validates a deploy artifact. On failure returns false with the
// reference's error message in *why.
bool load_artifact(const std::string &path, Json *config,
                   std::map<std::string, NamedTensor> *tensors, std::string *why);

} // namespace mu
