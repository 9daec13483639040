// candy_cuda.hpp -- C++ host layer over the C ABI (include/candyq.h).
//
// candy's host code is Go; where no Go toolchain is available this header is the compiled-language
// mirror of the slice of candy's backend interface that the quantized linear uses, with the same
// names and error behaviour, so that a C++ (or cgo-via-C++) host can use the library without
// touching raw status codes:
//   candy::cuda::Device    ~ candy.BackendDevice[float32]   (device.go:49-82)
//   candy::cuda::Storage   ~ candy.BackendStorage[float32]  (backend.go:4-238): Data, Clone, MatMul
//   candy::cuda::QStorage  -- the block-quantized weight storage candy lacks
//   candy::cuda::QLinear   ~ nn.Linear (nn/linear.go:11-112) with a quantized weight
// Every failure is a std::runtime_error whose text follows the reference's "<op>: <reason>" style.
#pragma once

#include <cstdint>
#include <memory>
#include <stdexcept>
#include <string>
#include <utility>
#include <vector>

#include "candyq.h"

namespace candy {
namespace cuda {

class Device;

inline void check(cq_ctx *ctx, cq_status s, const char *op) {
    if (s == CQ_OK) return;
    std::string msg = std::string(op) + ": " + cq_status_string(s);
    if (ctx) {
        const char *detail = cq_last_error(ctx);
        if (detail && *detail) msg += std::string(": ") + detail;
    }
    throw std::runtime_error(msg);
}

class Device : public std::enable_shared_from_this<Device> {
  public:
    static std::shared_ptr<Device> open(int ordinal = 0) {
        cq_ctx *ctx = nullptr;
        check(nullptr, cq_ctx_create(ordinal, &ctx), "cuda: create context");
        return std::shared_ptr<Device>(new Device(ctx, ordinal));
    }
    ~Device() {
        if (ctx_) cq_ctx_destroy(ctx_);
    }
    Device(const Device &) = delete;
    Device &operator=(const Device &) = delete;

    const char *location() const { return "gpu"; }                                   // BackendDevice.Location
    bool is_same(const Device &o) const { return o.ordinal_ == ordinal_; }           // BackendDevice.IsSame
    void synchronize() { check(ctx_, cq_synchronize(ctx_), "cuda: synchronize"); }   // BackendDevice.Synchronize
    cq_ctx *ctx() const { return ctx_; }
    int ordinal() const { return ordinal_; }

    void *malloc(size_t bytes) {
        void *p = nullptr;
        check(ctx_, cq_malloc(ctx_, bytes, &p), "cuda: alloc");
        return p;
    }
    void free(void *p) noexcept {
        if (p) cq_free(ctx_, p);
    }

  private:
    Device(cq_ctx *ctx, int ordinal) : ctx_(ctx), ordinal_(ordinal) {}
    cq_ctx *ctx_;
    int ordinal_;
};

class QStorage;

class Storage {
  public:
    // BackendDevice.StorageFromSlice / Alloc / Zeros
    static Storage from_slice(std::shared_ptr<Device> dev, const std::vector<float> &data) {
        Storage s(dev, data.size());
        if (!data.empty()) check(dev->ctx(), cq_memcpy_h2d(dev->ctx(), s.ptr_, data.data(), 4 * data.size()), "cuda: storage from slice");
        return s;
    }
    static Storage alloc(std::shared_ptr<Device> dev, size_t numel) { return Storage(dev, numel); }
    static Storage zeros(std::shared_ptr<Device> dev, size_t numel) {
        Storage s(dev, numel);
        check(dev->ctx(), cq_memset(dev->ctx(), s.ptr_, 0, 4 * numel), "cuda: zeros");
        return s;
    }
    Storage(Storage &&o) noexcept : dev_(std::move(o.dev_)), ptr_(o.ptr_), numel_(o.numel_) { o.ptr_ = nullptr; }
    Storage &operator=(Storage &&o) noexcept {
        if (this != &o) {
            release();
            dev_ = std::move(o.dev_), ptr_ = o.ptr_, numel_ = o.numel_, o.ptr_ = nullptr;
        }
        return *this;
    }
    Storage(const Storage &) = delete;
    Storage &operator=(const Storage &) = delete;
    ~Storage() { release(); }

    std::vector<float> data() const {  // BackendStorage.Data: a host copy
        std::vector<float> out(numel_);
        if (numel_) check(dev_->ctx(), cq_memcpy_d2h(dev_->ctx(), out.data(), ptr_, 4 * numel_), "cuda: data");
        return out;
    }
    Storage clone() const {  // BackendStorage.Clone
        Storage s(dev_, numel_);
        check(dev_->ctx(), cq_memcpy_d2d(dev_->ctx(), s.ptr_, ptr_, 4 * numel_), "cuda: clone");
        return s;
    }
    // BackendStorage.MatMul for a quantized right-hand side viewed as W^T [k,n]; this = [b*m, k].
    Storage matmul(const QStorage &rhs, int64_t b, int64_t m, int64_t n, int64_t k, int actmode = CQ_ACT_F32) const;

    float *ptr() const { return static_cast<float *>(ptr_); }
    size_t numel() const { return numel_; }
    const std::shared_ptr<Device> &device() const { return dev_; }  // BackendStorage.Device

  private:
    Storage(std::shared_ptr<Device> dev, size_t numel) : dev_(std::move(dev)), ptr_(nullptr), numel_(numel) {
        ptr_ = dev_->malloc(4 * (numel ? numel : 1));
    }
    void release() noexcept {
        if (ptr_ && dev_) dev_->free(ptr_);
        ptr_ = nullptr;
    }
    std::shared_ptr<Device> dev_;
    void *ptr_;
    size_t numel_;
};

class QStorage {
  public:
    // W[n,k] as n*k/32 blocks of `qtype` (host bytes, the reference's own layout).
    static QStorage from_blocks(std::shared_ptr<Device> dev, int qtype, int order, int64_t n, int64_t k, const std::vector<uint8_t> &blocks) {
        const size_t want = cq_blocks_bytes(qtype, n, k);
        if (want == 0) throw std::runtime_error("qstorage: k must be a positive multiple of 32 and the format Q4_0 or Q8_0");
        if (blocks.size() != want) throw std::runtime_error("qstorage: byte count does not match n*k/32 blocks");
        QStorage q(dev, qtype, order, n, k, want);
        check(dev->ctx(), cq_memcpy_h2d(dev->ctx(), q.ptr_, blocks.data(), want), "qstorage: upload");
        return q;
    }
    // Quantizes f32 W[n,k] on the GPU (arithmetic of the reference's quantizers, quantized.metal:4091-4214).
    static QStorage quantize(std::shared_ptr<Device> dev, int qtype, int order, int64_t n, int64_t k, const std::vector<float> &w) {
        const size_t want = cq_blocks_bytes(qtype, n, k);
        if (want == 0) throw std::runtime_error("qstorage: k must be a positive multiple of 32 and the format Q4_0 or Q8_0");
        if ((int64_t)w.size() != n * k) throw std::runtime_error("qstorage: weight size does not match n*k");
        Storage src = Storage::from_slice(dev, w);
        QStorage q(dev, qtype, order, n, k, want);
        check(dev->ctx(), cq_quantize_rows(dev->ctx(), qtype, order, src.ptr(), n, k, q.ptr_), "qstorage: quantize");
        dev->synchronize();  // src is released on return
        return q;
    }
    QStorage(QStorage &&o) noexcept : dev_(std::move(o.dev_)), ptr_(o.ptr_), bytes_(o.bytes_), qtype(o.qtype), order(o.order), n(o.n), k(o.k) {
        o.ptr_ = nullptr;
    }
    QStorage(const QStorage &) = delete;
    ~QStorage() {
        if (ptr_ && dev_) dev_->free(ptr_);
    }
    Storage dequantize() const {
        Storage out = Storage::alloc(dev_, (size_t)(n * k));
        check(dev_->ctx(), cq_dequantize(dev_->ctx(), qtype, order, ptr_, n * (k / 32), out.ptr()), "qstorage: dequantize");
        return out;
    }
    std::vector<uint8_t> data() const {
        std::vector<uint8_t> out(bytes_);
        check(dev_->ctx(), cq_memcpy_d2h(dev_->ctx(), out.data(), ptr_, bytes_), "qstorage: data");
        return out;
    }
    const void *ptr() const { return ptr_; }
    const std::shared_ptr<Device> &device() const { return dev_; }

  private:
    QStorage(std::shared_ptr<Device> dev, int qt, int ord, int64_t n_, int64_t k_, size_t bytes)
        : dev_(std::move(dev)), ptr_(nullptr), bytes_(bytes), qtype(qt), order(ord), n(n_), k(k_) {
        ptr_ = dev_->malloc(bytes);
    }
    std::shared_ptr<Device> dev_;
    void *ptr_;
    size_t bytes_;

  public:
    const int qtype, order;
    const int64_t n, k;
};

inline Storage Storage::matmul(const QStorage &rhs, int64_t b, int64_t m, int64_t n, int64_t k, int actmode) const {
    if (b < 1 || m < 1) throw std::runtime_error("matmul forward: bad batch or row count");
    if (k != rhs.k)
        throw std::runtime_error("matmul forward: inner dims mismatch: " + std::to_string(k) + " vs " + std::to_string(rhs.k));
    if (n != rhs.n) throw std::runtime_error("matmul forward: output dims mismatch: " + std::to_string(n) + " vs " + std::to_string(rhs.n));
    if ((int64_t)numel_ < b * m * k) throw std::runtime_error("matmul forward: lhs storage smaller than b*m*k");
    Storage out = Storage::alloc(dev_, (size_t)(b * m * n));
    check(dev_->ctx(), cq_qmatmul(dev_->ctx(), rhs.qtype, rhs.order, actmode, ptr(), b * m, k, k, rhs.ptr(), n, out.ptr(), n),
          "matmul forward: failed to matmul");
    return out;
}

// y = x W^T (+ b) for a contiguous x of shape [dims..., in]: nn.Linear.Forward's contiguous branch
// (nn/linear.go:72-92).  Wide batches (more than 8 rows) use the tensor-core mode unless told otherwise.
class QLinear {
  public:
    explicit QLinear(QStorage w, std::vector<float> bias = {}) : w_(std::move(w)), bias_(std::move(bias)) {
        if (!bias_.empty() && (int64_t)bias_.size() != w_.n) throw std::runtime_error("linear: bias shape must be [out]");
    }
    std::vector<float> forward(const std::vector<float> &x, const std::vector<int64_t> &dims, int actmode = -1) const {
        if (dims.size() < 2) throw std::runtime_error("linear: input rank must be >= 2, got " + std::to_string(dims.size()));
        int64_t rows = 1;
        for (size_t i = 0; i + 1 < dims.size(); ++i) rows *= dims[i];
        const int64_t k = dims.back();
        if ((int64_t)x.size() != rows * k) throw std::runtime_error("linear: failed to reshape input: size does not match dims");
        if (k != w_.k)
            throw std::runtime_error("linear: failed to matmul: matmul forward: inner dims mismatch: " + std::to_string(k) + " vs " +
                                     std::to_string(w_.k));
        if (actmode < 0) actmode = rows > 8 ? CQ_ACT_F16 : CQ_ACT_F32;
        Storage xs = Storage::from_slice(w_.device(), x);
        if (bias_.empty()) return xs.matmul(w_, 1, rows, w_.n, k, actmode).data();
        // BroadcastAdd (nn/linear.go:105-110) happens on the device, in the matmul's epilogue where its kernel has one
        if (!bias_dev_) bias_dev_.reset(new Storage(Storage::from_slice(w_.device(), bias_)));
        Storage out = Storage::alloc(w_.device(), (size_t)(rows * w_.n));
        check(w_.device()->ctx(),
              cq_qlinear(w_.device()->ctx(), w_.qtype, w_.order, actmode, xs.ptr(), rows, k, k, w_.ptr(), w_.n, bias_dev_->ptr(), out.ptr(), w_.n),
              "linear: failed to matmul");
        return out.data();
    }
    const QStorage &weight() const { return w_; }

  private:
    QStorage w_;
    std::vector<float> bias_;
    mutable std::unique_ptr<Storage> bias_dev_;  // the bias, uploaded on first use
};

}  // namespace cuda
}  // namespace candy
