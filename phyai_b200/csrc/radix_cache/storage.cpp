// Payload stores for the lower cache tiers: a hash map in memory and a slotted file on disk.
// Reference: phyai-ext/csrc/radix_cache/storage_backend.h:31-110.
#include <fcntl.h>
#include <sys/stat.h>
#include <unistd.h>

#include <cerrno>
#include <cstring>

#include "radix_cache.h"

namespace pbc {

namespace {

class MemoryBackend final : public StorageBackend {
 public:
  explicit MemoryBackend(std::size_t unit_bytes) : unit_(unit_bytes) {}
  std::string name() const override { return "memory"; }
  std::size_t unit_bytes() const override { return unit_; }
  bool write(std::uint64_t key, std::string_view payload) override {
    if (unit_ == 0 || payload.size() % unit_) return false;
    std::lock_guard<std::mutex> g(mu_);
    map_[key] = std::string(payload);
    return true;
  }
  std::optional<std::string> read(std::uint64_t key) override {
    std::lock_guard<std::mutex> g(mu_);
    auto it = map_.find(key);
    if (it == map_.end()) return std::nullopt;
    return it->second;
  }
  bool contains(std::uint64_t key) const override { std::lock_guard<std::mutex> g(mu_); return map_.count(key) > 0; }
  bool erase(std::uint64_t key) override { std::lock_guard<std::mutex> g(mu_); return map_.erase(key) > 0; }
  std::size_t entries() const override { std::lock_guard<std::mutex> g(mu_); return map_.size(); }
  void drain() override {}
 private:
  std::size_t unit_;
  mutable std::mutex mu_;
  std::unordered_map<std::uint64_t, std::string> map_;
};

// One file, append-only extents with a free list of erased extents of equal length.
class FileBackend final : public StorageBackend {
 public:
  FileBackend(const std::string& path, std::size_t unit_bytes) : unit_(unit_bytes), path_(path) {
    fd_ = ::open(path.c_str(), O_RDWR | O_CREAT | O_TRUNC, 0600);
    if (fd_ < 0) throw UsageError("cannot open " + path + ": " + std::strerror(errno));
  }
  ~FileBackend() override { if (fd_ >= 0) ::close(fd_); }
  std::string name() const override { return "file:" + path_; }
  std::size_t unit_bytes() const override { return unit_; }
  bool write(std::uint64_t key, std::string_view payload) override {
    if (unit_ == 0 || payload.size() % unit_) return false;
    std::lock_guard<std::mutex> g(mu_);
    erase_locked(key);
    off_t off = -1;
    auto fl = free_.find(payload.size());
    if (fl != free_.end() && !fl->second.empty()) { off = fl->second.back(); fl->second.pop_back(); }
    else { off = end_; end_ += off_t(payload.size()); }
    std::size_t done = 0;
    while (done < payload.size()) {
      const ssize_t w = ::pwrite(fd_, payload.data() + done, payload.size() - done, off + off_t(done));
      if (w < 0) { if (errno == EINTR) continue; return false; }
      done += std::size_t(w);
    }
    index_[key] = {off, payload.size()};
    return true;
  }
  std::optional<std::string> read(std::uint64_t key) override {
    std::lock_guard<std::mutex> g(mu_);
    auto it = index_.find(key);
    if (it == index_.end()) return std::nullopt;
    std::string out(it->second.len, '\0');
    std::size_t done = 0;
    while (done < out.size()) {
      const ssize_t r = ::pread(fd_, out.data() + done, out.size() - done, it->second.off + off_t(done));
      if (r < 0) { if (errno == EINTR) continue; return std::nullopt; }
      if (r == 0) return std::nullopt;
      done += std::size_t(r);
    }
    return out;
  }
  bool contains(std::uint64_t key) const override { std::lock_guard<std::mutex> g(mu_); return index_.count(key) > 0; }
  bool erase(std::uint64_t key) override { std::lock_guard<std::mutex> g(mu_); return erase_locked(key); }
  std::size_t entries() const override { std::lock_guard<std::mutex> g(mu_); return index_.size(); }
  void drain() override { std::lock_guard<std::mutex> g(mu_); ::fsync(fd_); }
 private:
  struct Extent { off_t off; std::size_t len; };
  bool erase_locked(std::uint64_t key) {
    auto it = index_.find(key);
    if (it == index_.end()) return false;
    free_[it->second.len].push_back(it->second.off);
    index_.erase(it);
    return true;
  }
  std::size_t unit_;
  std::string path_;
  int fd_ = -1;
  off_t end_ = 0;
  mutable std::mutex mu_;
  std::unordered_map<std::uint64_t, Extent> index_;
  std::unordered_map<std::size_t, std::vector<off_t>> free_;
};

}  // namespace

std::shared_ptr<StorageBackend> make_memory_backend(std::size_t unit_bytes) { return std::make_shared<MemoryBackend>(unit_bytes); }
std::shared_ptr<StorageBackend> make_file_backend(const std::string& path, std::size_t unit_bytes) {
  return std::make_shared<FileBackend>(path, unit_bytes);
}

}  // namespace pbc
