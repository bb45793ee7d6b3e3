// safetensors.hpp — read-only access to a model folder of the second container the engine loads: config.json (a JSON
// object) + model.safetensors (8-byte little-endian header length, that many bytes of JSON mapping tensor name ->
// {dtype, shape, data_offsets}, then the raw little-endian data). Written from the format definition; the GGUF reader
// (gguf.hpp) stays the container of the quantized LLaMA path.
#pragma once
#include <cstdint>
#include <map>
#include <memory>
#include <string>
#include <vector>

namespace b200 {

// a JSON value: null | bool | number | string | array | object. Objects keep insertion order of no interest: a map.
struct Json {
    enum Kind { Null, Bool, Num, Str, Arr, Obj } kind = Null;
    bool b = false;
    double num = 0;
    std::string str;
    std::vector<Json> arr;
    std::map<std::string, Json> obj;

    bool is_null() const { return kind == Null; }
    bool has(const std::string & k) const { return kind == Obj && obj.count(k) > 0 && !obj.at(k).is_null(); }
    // required members throw std::runtime_error naming the key
    const Json & at(const std::string & k) const;
    double  number(const std::string & k) const;
    double  number(const std::string & k, double def) const { return has(k) ? number(k) : def; }
    int64_t integer(const std::string & k) const;
    int64_t integer(const std::string & k, int64_t def) const { return has(k) ? integer(k) : def; }
    std::string string(const std::string & k, const std::string & def) const;
};
Json json_parse(const char * text, size_t n);     // throws std::runtime_error with the byte offset
Json json_parse_file(const std::string & path);

enum st_dtype { ST_BF16 = 0, ST_F32, ST_F16, ST_I32, ST_OTHER };

struct st_tensor {
    std::string name;
    st_dtype dtype = ST_OTHER;
    std::vector<int64_t> shape;
    const uint8_t * data = nullptr;
    uint64_t nbytes = 0;
    int64_t numel() const { int64_t n = 1; for (int64_t d : shape) n *= d; return n; }
};

struct safetensors_file {
    int fd = -1;
    const uint8_t * base = nullptr;
    uint64_t size = 0;
    std::map<std::string, st_tensor> tensors;
    ~safetensors_file();
    void open(const std::string & path);           // throws
    const st_tensor * find(const std::string & name) const;
    // the tensor as float32 (bfloat16 / float16 / float32 sources), shape checked against `shape` (throws)
    std::vector<float> read_f32(const std::string & name, const std::vector<int64_t> & shape) const;
};

// "<dir>/config.json" exists (or path itself is such a file): the folder container, not a GGUF file
bool is_model_dir(const std::string & path, std::string * dir_out);

}  // namespace b200
