// Stand-in for nanoarrow.hpp: owning wrappers around the Arrow C data / stream
// structs (release on destruction, move-only) and the exception type, as far as the
// reference framework's Arrow wrapper uses them. Built only for the offline
// benchmark build of the reference.
#ifndef NANOARROW_STANDIN_HPP_
#define NANOARROW_STANDIN_HPP_

#include <cstring>
#include <stdexcept>
#include <string>

#include "nanoarrow/nanoarrow.h"

namespace nanoarrow {

class Exception : public std::runtime_error {
 public:
  explicit Exception(const std::string& msg) : std::runtime_error(msg) {}
};

namespace internal {

// Takes ownership by moving the C struct's contents out of the source (which is
// marked released), the convention of the Arrow C data interface.
template <typename T>
class Unique {
 public:
  Unique() { std::memset(&data_, 0, sizeof(data_)); }
  explicit Unique(T* src) {
    std::memcpy(&data_, src, sizeof(T));
    src->release = nullptr;
  }
  Unique(Unique&& rhs) noexcept {
    std::memcpy(&data_, &rhs.data_, sizeof(T));
    rhs.data_.release = nullptr;
  }
  Unique& operator=(Unique&& rhs) noexcept {
    if (this != &rhs) {
      reset();
      std::memcpy(&data_, &rhs.data_, sizeof(T));
      rhs.data_.release = nullptr;
    }
    return *this;
  }
  Unique(const Unique&) = delete;
  Unique& operator=(const Unique&) = delete;
  ~Unique() { reset(); }

  void reset() {
    if (data_.release != nullptr) data_.release(&data_);
    data_.release = nullptr;
  }
  T* get() noexcept { return &data_; }
  const T* get() const noexcept { return &data_; }
  T* operator->() noexcept { return &data_; }
  const T* operator->() const noexcept { return &data_; }

 private:
  T data_;
};

}  // namespace internal

using UniqueSchema = internal::Unique<struct ArrowSchema>;
using UniqueArray = internal::Unique<struct ArrowArray>;
using UniqueArrayStream = internal::Unique<struct ArrowArrayStream>;

}  // namespace nanoarrow

#endif  // NANOARROW_STANDIN_HPP_
