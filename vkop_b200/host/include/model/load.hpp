// Reader of the reference's binary model file (.vkopbin), the format its ONNX converter writes and
// model/load.cpp:98-285 parses.  Same namespace, class and field names as model/load.hpp, so that code
// written against vkop::load::VkModel compiles unchanged.
//
// File layout (all integers little-endian; a string is a u32 length and its bytes; dims are a u32 count
// and that many u32):
//   inputs        u32 n, then n x (name, dims)
//   outputs       the same
//   nodes         u32 n, then n x (op_type, name, attributes, inputs, outputs, dependencies, dependents)
//                 attributes: u32 n, then n x (key, u8 tag, value): tag 0 string, 1 int64, 2 float32,
//                 3 list of u32, 4 list of float32 (load.hpp:241-275); lists print as "[a, b, ...]"
//                 inputs / outputs: as the model's; dependencies / dependents: u32 n, then n names
//   initializers  u32 n, then n x (name, dtype name, dims, i64 byte size, the bytes)
//   levels        u32 n, then n x (u32 m, then m node names): nodes that may run side by side
// The initializer bytes are copied into one block, each at a 64-byte aligned offset, as the reference does.
// Not reproduced: the reference's unpacking of "unified_*" and "rgba_conversion_*" initializers, which
// describe weight packings of its image-based convolution path (load.cpp:186-285).
#ifndef VKOP_HOST_MODEL_LOAD_HPP_
#define VKOP_HOST_MODEL_LOAD_HPP_

#include <cstdint>
#include <cstring>
#include <fstream>
#include <iterator>
#include <sstream>
#include <stdexcept>
#include <string>
#include <unordered_map>
#include <unordered_set>
#include <vector>

namespace vkop {
namespace load {

struct Shape {
    std::string name;
    std::vector<uint32_t> dims;
};

struct Node {
    std::string op_type, name;
    std::unordered_map<std::string, std::string> attributes;
    std::vector<Shape> inputs, outputs;
    std::unordered_set<std::string> dependencies, dependents;
};

struct Initializer {
    std::string name, dtype;
    std::vector<uint32_t> dims;
    int64_t byte_size = 0;
};

class VkModel {
  public:
    explicit VkModel(const std::string &file_path) { loadFromBinary(file_path); }

    std::vector<Shape> inputs, outputs;
    std::vector<Node> nodes;
    std::unordered_map<std::string, Initializer> initializers;
    std::unordered_map<std::string, size_t> initializer_offsets;
    std::vector<uint8_t> initializer_memory;
    std::vector<std::vector<std::string>> concurrent_execution_levels;

    const uint8_t *initializer_data(const std::string &name) const {
        auto it = initializer_offsets.find(name);
        return it == initializer_offsets.end() ? nullptr : initializer_memory.data() + it->second;
    }

    // One line per input, output, node, initializer and level.
    std::string describe() const {
        std::ostringstream o;
        auto dims = [&](const std::vector<uint32_t> &d) {
            o << "[";
            for (size_t i = 0; i < d.size(); i++)
                o << (i ? "," : "") << d[i];
            o << "]";
        };
        for (const auto &s : inputs) {
            o << "input " << s.name << " ";
            dims(s.dims);
            o << "\n";
        }
        for (const auto &s : outputs) {
            o << "output " << s.name << " ";
            dims(s.dims);
            o << "\n";
        }
        for (const auto &n : nodes) {
            o << "node " << n.op_type << " " << n.name << " in";
            for (const auto &s : n.inputs)
                o << " " << s.name;
            o << " out";
            for (const auto &s : n.outputs)
                o << " " << s.name;
            o << " attrs " << n.attributes.size() << "\n";
        }
        for (const auto &kv : initializers) {
            o << "initializer " << kv.first << " " << kv.second.dtype << " ";
            dims(kv.second.dims);
            o << " " << kv.second.byte_size << "\n";
        }
        for (size_t l = 0; l < concurrent_execution_levels.size(); l++) {
            o << "level " << l;
            for (const auto &n : concurrent_execution_levels[l])
                o << " " << n;
            o << "\n";
        }
        return o.str();
    }

  private:
    // A cursor over the file's bytes; every read is checked against the end.
    class Cursor {
      public:
        Cursor(const uint8_t *p, size_t n) : p_(p), end_(p + n) {}
        template <typename T>
        T scalar(const char *what) {
            need(sizeof(T), what);
            T v;
            std::memcpy(&v, p_, sizeof(T));
            p_ += sizeof(T);
            return v;
        }
        uint32_t count(const char *what) {
            const uint32_t n = scalar<uint32_t>(what);
            if (n > static_cast<size_t>(end_ - p_))  // every counted item takes at least a byte
                throw std::runtime_error(std::string("vkopbin: implausible count for ") + what);
            return n;
        }
        std::string str() {
            const uint32_t n = count("string");
            std::string s(reinterpret_cast<const char *>(p_), n);
            p_ += n;
            return s;
        }
        std::vector<uint32_t> dims() {
            const uint32_t n = count("dims");
            need(static_cast<size_t>(n) * 4, "dims");
            std::vector<uint32_t> d(n);
            for (auto &v : d)
                v = scalar<uint32_t>("dim");
            return d;
        }
        std::vector<Shape> shapes() {
            const uint32_t n = count("shape list");
            std::vector<Shape> out(n);
            for (auto &s : out) {
                s.name = str();
                s.dims = dims();
            }
            return out;
        }
        std::unordered_set<std::string> names() {
            const uint32_t n = count("name list");
            std::unordered_set<std::string> out;
            for (uint32_t i = 0; i < n; i++)
                out.insert(str());
            return out;
        }
        template <typename T>
        std::string list_text(const char *what) {
            const uint32_t n = count(what);
            std::string s = "[";
            for (uint32_t i = 0; i < n; i++)
                s += (i ? ", " : "") + std::to_string(scalar<T>(what));
            return s + "]";
        }
        std::unordered_map<std::string, std::string> dict() {
            const uint32_t n = count("attributes");
            std::unordered_map<std::string, std::string> d;
            for (uint32_t i = 0; i < n; i++) {
                const std::string key = str();
                const uint8_t tag = scalar<uint8_t>("attribute tag");
                switch (tag) {
                case 0: d[key] = str(); break;
                case 1: d[key] = std::to_string(scalar<int64_t>("int attribute")); break;
                case 2: d[key] = std::to_string(scalar<float>("float attribute")); break;
                case 3: d[key] = list_text<uint32_t>("int list attribute"); break;
                case 4: d[key] = list_text<float>("float list attribute"); break;
                default: throw std::runtime_error("vkopbin: unknown attribute tag " + std::to_string(tag));
                }
            }
            return d;
        }
        const uint8_t *skip(size_t n, const char *what) {
            need(n, what);
            const uint8_t *at = p_;
            p_ += n;
            return at;
        }

      private:
        void need(size_t n, const char *what) const {
            if (n > static_cast<size_t>(end_ - p_))
                throw std::runtime_error(std::string("vkopbin: unexpected end of file in ") + what);
        }
        const uint8_t *p_, *end_;
    };

    void loadFromBinary(const std::string &file_path) {
        std::ifstream f(file_path, std::ios::binary);
        if (!f)
            throw std::runtime_error("Failed to open model file: " + file_path);
        const std::vector<uint8_t> bytes((std::istreambuf_iterator<char>(f)), std::istreambuf_iterator<char>());
        Cursor c(bytes.data(), bytes.size());
        inputs = c.shapes();
        outputs = c.shapes();
        const uint32_t num_nodes = c.count("nodes");
        nodes.reserve(num_nodes);
        for (uint32_t i = 0; i < num_nodes; i++) {
            Node n;
            n.op_type = c.str();
            n.name = c.str();
            n.attributes = c.dict();
            n.inputs = c.shapes();
            n.outputs = c.shapes();
            n.dependencies = c.names();
            n.dependents = c.names();
            nodes.push_back(std::move(n));
        }
        const uint32_t num_init = c.count("initializers");
        constexpr size_t kAlign = 64;
        struct Blob {
            const uint8_t *at;
            size_t offset, size;
        };
        std::vector<Blob> blobs;
        size_t total = 0;
        for (uint32_t i = 0; i < num_init; i++) {
            Initializer in;
            in.name = c.str();
            in.dtype = c.str();
            in.dims = c.dims();
            in.byte_size = c.scalar<int64_t>("initializer size");
            if (in.byte_size < 0)
                throw std::runtime_error("vkopbin: negative initializer size");
            const size_t size = static_cast<size_t>(in.byte_size);
            const uint8_t *at = c.skip(size, "initializer data");
            const size_t off = (total + kAlign - 1) / kAlign * kAlign;
            initializer_offsets[in.name] = off;
            total = off + size;
            blobs.push_back(Blob{at, off, size});
            initializers[in.name] = std::move(in);
        }
        initializer_memory.assign(total, 0);
        for (const Blob &b : blobs)
            std::memcpy(initializer_memory.data() + b.offset, b.at, b.size);
        const uint32_t num_levels = c.count("levels");
        concurrent_execution_levels.resize(num_levels);
        for (auto &level : concurrent_execution_levels) {
            const uint32_t m = c.count("level");
            level.reserve(m);
            for (uint32_t j = 0; j < m; j++)
                level.push_back(c.str());
        }
    }

};

}  // namespace load
}  // namespace vkop
#endif  // VKOP_HOST_MODEL_LOAD_HPP_
