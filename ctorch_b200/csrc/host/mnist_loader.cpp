// IDX reader (mnist/mnist_loader.cpp:7-73 of the reference): big-endian int32 magic (2051 images,
// 2049 labels), big-endian int32 extents, then one unsigned byte per pixel / label.  Pixels become
// pixel / 255.0f (:38-40), labels become floats holding the integer (:113-115).
#include "mnist_loader.h"

#include <cstdio>
#include <stdexcept>

#include "ctorch_b200.h"

namespace ctorch {

namespace {
int be32(const unsigned char* p) { return static_cast<int>((static_cast<unsigned>(p[0]) << 24) | (static_cast<unsigned>(p[1]) << 16) | (static_cast<unsigned>(p[2]) << 8) | p[3]); }
}  // namespace

MNISTLoader::MNISTLoader(const std::string& dir, DeviceType dev) : data_dir(dir), device(dev) {}

void MNISTLoader::read_idx(const std::string& filename, int expected_magic, std::vector<unsigned char>& bytes, std::vector<int>& dims) const {
    const std::string path = data_dir + "/" + filename;
    std::FILE* f = std::fopen(path.c_str(), "rb");
    if (!f) throw std::runtime_error("cannot open file: " + filename);
    unsigned char head[16];
    const int n_dims = expected_magic == 2051 ? 3 : 1;
    if (std::fread(head, 1, 4, f) != 4) {
        std::fclose(f);
        throw std::runtime_error("file too short for an IDX header: " + filename);
    }
    if (be32(head) != expected_magic) {
        std::fclose(f);
        throw std::runtime_error(expected_magic == 2051 ? "not an IDX image file (magic number is not 2051): " + filename
                                                        : "not an IDX label file (magic number is not 2049): " + filename);
    }
    if (std::fread(head + 4, 1, 4 * static_cast<size_t>(n_dims), f) != 4 * static_cast<size_t>(n_dims)) {
        std::fclose(f);
        throw std::runtime_error("file too short for an IDX header: " + filename);
    }
    dims.clear();
    size_t count = 1;
    for (int i = 0; i < n_dims; ++i) {
        const int d = be32(head + 4 + 4 * i);
        if (d < 0) {
            std::fclose(f);
            throw std::runtime_error("negative extent in the IDX header: " + filename);
        }
        dims.push_back(d);
        count *= static_cast<size_t>(d);
    }
    bytes.resize(count);
    const size_t got = count ? std::fread(bytes.data(), 1, count, f) : 0;
    std::fclose(f);
    // (the reference keeps going on a short file and leaves the missing pixels undefined)
    if (got != count) throw std::runtime_error("IDX payload shorter than its header announces: " + filename);
}

Tensor MNISTLoader::to_tensor(const std::vector<unsigned char>& bytes, const std::vector<size_t>& shape, float divisor) const {
    Tensor t(ShapeTag{}, shape, DType::kFloat, device, false);
    const size_t n = bytes.size();
    if (n == 0) return t;
    if (device == DeviceType::kCUDA) {
        // bytes -> page-locked memory -> device -> floats on the device
        void* pinned = nullptr;
        void* dev_bytes = nullptr;
        cuda_check(ctk_malloc_host(&pinned, n), "MNISTLoader: page-locked buffer");
        std::memcpy(pinned, bytes.data(), n);
        int rc = ctk_malloc(&dev_bytes, n);
        if (!rc) rc = ctk_memcpy_h2d(dev_bytes, pinned, n, current_stream());
        if (!rc) rc = ctk_u8_to_f32(static_cast<const uint8_t*>(dev_bytes), static_cast<int64_t>(n), divisor, t.data<float>(), current_stream());
        if (!rc) rc = current_stream() ? ctk_stream_sync(current_stream()) : ctk_device_sync();
        if (dev_bytes) ctk_free(dev_bytes);
        ctk_free_host(pinned);
        cuda_check(rc, "MNISTLoader: upload");
    } else {
        float* out = t.data<float>();
        for (size_t i = 0; i < n; ++i) out[i] = bytes[i] / divisor;
    }
    return t;
}

void MNISTLoader::load(const std::string& image_file, const std::string& label_file, Tensor& images, Tensor& labels) {
    std::vector<unsigned char> pixels, labs;
    std::vector<int> idims, ldims;
    read_idx(image_file, 2051, pixels, idims);
    read_idx(label_file, 2049, labs, ldims);
    images = to_tensor(pixels, {static_cast<size_t>(idims[0]), static_cast<size_t>(idims[1]) * static_cast<size_t>(idims[2])}, 255.0f);
    labels = to_tensor(labs, {static_cast<size_t>(ldims[0])}, 1.0f);
}

void MNISTLoader::load_training_data(Tensor& images, Tensor& labels) { load("train-images-idx3-ubyte", "train-labels-idx1-ubyte", images, labels); }
void MNISTLoader::load_test_data(Tensor& images, Tensor& labels) { load("t10k-images-idx3-ubyte", "t10k-labels-idx1-ubyte", images, labels); }

}  // namespace ctorch
