// Test infrastructure, not the product: a C wrapper over the UNMODIFIED reference weight-file code
// (src/serialization.cpp: TensorFileFormat, the .nve container; NumpyTensorFileFormat;
// BinaryTensorFileFormat), compiled where the reference checkout lies.  Used to write golden files
// and to read back what this repository's own reader / writer (weight_files.py) produce.
#include <cstdio>
#include <cstring>
#include <memory>
#include <string>
#include <vector>

#include "serialization.hpp"

namespace {

thread_local std::string g_error;

// Read/write stream over a stdio file (the reference ships only an input stream; its Python
// binding supplies the output side).
class FileStream : public nve::StreamWrapperBase {
 public:
  FileStream(const char* path, const char* mode) : f_(std::fopen(path, mode)) {}
  ~FileStream() override { if (f_) std::fclose(f_); }
  bool ok() const { return f_ != nullptr; }
  void write(const void* data, size_t size) override { std::fwrite(data, 1, size, f_); }
  uint64_t seek(uint64_t offset) override { std::fseek(f_, static_cast<long>(offset), SEEK_SET); return offset; }
  uint64_t tell() override { return static_cast<uint64_t>(std::ftell(f_)); }
  void flush() override { std::fflush(f_); }
  uint64_t read(void* data, size_t size) override { return std::fread(data, 1, size, f_); }
  uint64_t size() override {
    const long at = std::ftell(f_);
    std::fseek(f_, 0, SEEK_END);
    const long n = std::ftell(f_);
    std::fseek(f_, at, SEEK_SET);
    return static_cast<uint64_t>(n);
  }

 private:
  FILE* f_;
};

template <typename Fn>
int guarded(Fn&& fn) {
  try {
    fn();
    return 0;
  } catch (const std::exception& e) {
    g_error = e.what();
    return 1;
  }
}

}  // namespace

extern "C" {

const char* refser_last_error() { return g_error.c_str(); }

// Writes a .nve file holding `count` tensors: names[i], data[i] of rows[i] x cols[i] elements of
// elem_bytes[i].
int refser_write_nve(const char* path, int count, const uint64_t* names, const void* const* data,
                     const uint64_t* rows, const uint64_t* cols, const uint64_t* elem_bytes) {
  return guarded([&] {
    FileStream s(path, "wb+");
    if (!s.ok()) throw std::runtime_error("cannot open file for writing");
    nve::TensorFileFormat fmt;
    fmt.write_table_file_header(s);
    for (int i = 0; i < count; i++) {
      nve::TensorWrapper t;
      t.data = const_cast<void*>(data[i]);
      t.row = rows[i];
      t.col = cols[i];
      t.element_size_in_bytes = elem_bytes[i];
      fmt.write_tensor_to_stream(s, names[i], t);
    }
  });
}

// Reads tensor `name` (rows x cols x elem_bytes, which must match the stored size) into `out`.
int refser_read_nve(const char* path, uint64_t name, uint64_t rows, uint64_t cols, uint64_t elem_bytes, void* out) {
  return guarded([&] {
    FileStream s(path, "rb");
    if (!s.ok()) throw std::runtime_error("cannot open file");
    nve::TensorFileFormat fmt;
    nve::TensorWrapper t;
    t.data = out;
    t.row = rows;
    t.col = cols;
    t.element_size_in_bytes = elem_bytes;
    fmt.load_tensor_from_stream(s, name, t);
  });
}

// Shape of a .npy file as the reference parses it: rows and bytes per row.
int refser_numpy_info(const char* path, uint64_t* rows, uint64_t* row_bytes) {
  return guarded([&] {
    nve::NumpyTensorFileFormat f(std::make_shared<nve::InputFileStreamWrapper>(path));
    *rows = f.get_num_rows();
    *row_bytes = f.get_row_size_in_bytes();
  });
}

// Loads `rows` rows of a .npy file in two batches (the loader is a stream of batches).
int refser_numpy_load(const char* path, uint64_t rows, void* out) {
  return guarded([&] {
    nve::NumpyTensorFileFormat f(std::make_shared<nve::InputFileStreamWrapper>(path));
    f.reset();
    const uint64_t first = rows / 2;
    f.load_batch(first, out);
    f.load_batch(rows - first, static_cast<char*>(out) + first * f.get_row_size_in_bytes());
  });
}

// Rows of a raw binary table file with the given row size, and their bytes.
int refser_binary_load(const char* path, uint64_t row_bytes, uint64_t* rows, void* out, uint64_t out_rows) {
  return guarded([&] {
    nve::BinaryTensorFileFormat f(std::make_shared<nve::InputFileStreamWrapper>(path), row_bytes);
    *rows = f.get_num_rows();
    if (out != nullptr) {
      f.reset();
      f.load_batch(out_rows, out);
    }
  });
}

}  // extern "C"
