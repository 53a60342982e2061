// MNISTLoader: reader of the IDX files of the MNIST distribution, with the public surface of the
// reference's mnist/mnist_loader.h (constructor from a directory, load_training_data,
// load_test_data filling an [n, rows*cols] image tensor of pixel/255 and an [n] label tensor of
// floats) plus a target device.
//
// For DeviceType::kCUDA the file's bytes go to the device as they are (one read into page-locked
// memory, one copy) and are turned into floats there: a quarter of the PCIe traffic of uploading
// floats, and the /255 runs at HBM speed instead of one byte per ifstream::read call.
#pragma once
#include <string>
#include <vector>

#include "Tensor.h"

namespace ctorch {

class MNISTLoader {
    std::string data_dir;
    DeviceType device;

    // Parses one IDX file into `bytes` (the payload) and its dimensions; throws std::runtime_error if
    // the file cannot be opened, the magic number is wrong or the payload is shorter than announced.
    void read_idx(const std::string& filename, int expected_magic, std::vector<unsigned char>& bytes, std::vector<int>& dims) const;
    Tensor to_tensor(const std::vector<unsigned char>& bytes, const std::vector<size_t>& shape, float divisor) const;

public:
    explicit MNISTLoader(const std::string& dir, DeviceType device = DeviceType::kCPU);

    void load_training_data(Tensor& images, Tensor& labels);  // train-images-idx3-ubyte, train-labels-idx1-ubyte
    void load_test_data(Tensor& images, Tensor& labels);      // t10k-images-idx3-ubyte, t10k-labels-idx1-ubyte
    // Any image / label file pair of the directory.
    void load(const std::string& image_file, const std::string& label_file, Tensor& images, Tensor& labels);
};

}  // namespace ctorch
