// Test infrastructure only. Minimal stand-in for the third-party header <mio/mmap.hpp> (mandreyel/mio, pulled in by
// the reference through vcpkg and absent here), offering exactly what the reference's GGUF parser uses
// (include/gguf.hpp:183, src/gguf.cpp:173,195-211): a read-only mapping of a file built from its path, size(),
// data() and iteration as a contiguous range of char.
#pragma once

#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <cstddef>
#include <stdexcept>
#include <utility>

namespace mio {

class mmap_source {
   public:
    using value_type = char;
    using const_iterator = const char*;
    using iterator = const char*;

    mmap_source() = default;
    explicit mmap_source(const char* path) {
        const int fd = ::open(path, O_RDONLY);
        if (fd < 0) throw std::runtime_error("cannot open file");
        struct stat st {};
        if (::fstat(fd, &st) != 0) {
            ::close(fd);
            throw std::runtime_error("cannot stat file");
        }
        size_ = static_cast<std::size_t>(st.st_size);
        void* p = size_ ? ::mmap(nullptr, size_, PROT_READ, MAP_PRIVATE, fd, 0) : nullptr;
        ::close(fd);
        if (size_ && p == MAP_FAILED) throw std::runtime_error("cannot map file");
        data_ = static_cast<const char*>(p);
    }
    mmap_source(const mmap_source&) = delete;
    mmap_source& operator=(const mmap_source&) = delete;
    mmap_source(mmap_source&& o) noexcept : data_(std::exchange(o.data_, nullptr)), size_(std::exchange(o.size_, 0)) {}
    mmap_source& operator=(mmap_source&& o) noexcept {
        if (this != &o) {
            release();
            data_ = std::exchange(o.data_, nullptr);
            size_ = std::exchange(o.size_, 0);
        }
        return *this;
    }
    ~mmap_source() { release(); }

    [[nodiscard]] std::size_t size() const noexcept { return size_; }
    [[nodiscard]] const char* data() const noexcept { return data_; }
    [[nodiscard]] const char* begin() const noexcept { return data_; }
    [[nodiscard]] const char* end() const noexcept { return data_ + size_; }

   private:
    void release() noexcept {
        if (data_) ::munmap(const_cast<char*>(data_), size_);
        data_ = nullptr;
        size_ = 0;
    }
    const char* data_ = nullptr;
    std::size_t size_ = 0;
};

}  // namespace mio
