// Vocabulary types of the gradc host API: devices, dtypes, tags, index descriptors, op enums and GPTConfig.
// Same spelling and meaning as the reference's gradc/core/types.hpp:10-183 and gradc/backend/op_types.hpp:3-8,
// so that code written against GradCraft (train.cpp in particular) compiles unchanged.
#pragma once

#include <cstdint>
#include <iostream>
#include <optional>
#include <type_traits>
#include <utility>
#include <vector>

enum class UnaryOp { Identity, Neg, ReLU, Exp, Log, Sin, Cos, Square, Sqrt, Sigmoid, TanH, SiLU, GeLU, Cast };
enum class UnaryOpInPlace { ReLU, Neg, Exp, Log, Sin, Cos, Square, Sqrt, Sigmoid, TanH, SiLU, GeLU };
enum class BinaryOp { Add, Sub, Mul, Div, MatMul, EqMask, BReLU, BSigmoid, BTanH, BSiLU, BGeLU, BExp, BLog, BSin, BCos, BSquare, BSqrt };
enum class BinaryOpInPlace { Add, Sub, ISub, Mul, Div, IDiv, MatMul, GrThan };
enum class ReduceOp { Sum, Mean, Max, Min };
enum class ArgExtrOp { ArgMax, ArgMin };

namespace gradc {

enum class DType { Float32, Float64, Int32, Int64, Unknown };

template <typename T>
constexpr DType type_to_dtype() {
    if constexpr (std::is_same_v<T, float>) return DType::Float32;
    else if constexpr (std::is_same_v<T, double>) return DType::Float64;
    else if constexpr (std::is_same_v<T, int32_t>) return DType::Int32;
    else if constexpr (std::is_same_v<T, int64_t>) return DType::Int64;
    else return DType::Unknown;
}

template <typename T>
constexpr bool is_supported_tensor_type_v = std::is_same_v<T, int32_t> || std::is_same_v<T, int64_t> || std::is_same_v<T, float> || std::is_same_v<T, double>;

enum class DeviceType { CPU, CUDA };

struct Device {
    DeviceType type;
    int32_t index;
    constexpr Device(DeviceType t = DeviceType::CPU, int32_t i = -1) : type(t), index(i) {}
    constexpr bool is_cpu() const { return type == DeviceType::CPU; }
    constexpr bool is_cuda() const { return type == DeviceType::CUDA; }
    constexpr bool operator==(const Device& o) const { return is_cpu() ? o.is_cpu() : (o.type == type && o.index == index); }
    constexpr bool operator!=(const Device& o) const { return !(*this == o); }
    friend std::ostream& operator<<(std::ostream& os, const Device& d) {
        if (d.is_cpu()) return os << "CPU";
        return os << "CUDA:" << d.index;
    }
};

enum IndexType { Single, Range, All };

struct Slice {
    std::optional<int64_t> start, stop, step;
    Slice(std::optional<int64_t> a = std::nullopt, std::optional<int64_t> b = std::nullopt, std::optional<int64_t> c = std::nullopt) : start(a), stop(b), step(c) {}
};
struct AllSlice {};
inline constexpr AllSlice _ = AllSlice();

struct IndexDesc {
    IndexType m_type;
    int64_t m_single_val = 0;
    Slice m_slice_val;
    IndexDesc(int64_t v) : m_type(IndexType::Single), m_single_val(v) {}
    IndexDesc(int v) : m_type(IndexType::Single), m_single_val(v) {}
    IndexDesc(AllSlice) : m_type(IndexType::All) {}
    IndexDesc(Slice s) : m_type(IndexType::Range), m_slice_val(std::move(s)) {}
};

enum MatrixTensorOp { Normal, Transposed };

struct LazyTag {};
inline constexpr LazyTag lazy = LazyTag();
struct UninitializedTag {};
inline constexpr UninitializedTag uninitialized = UninitializedTag();

struct GPTConfig {
    int64_t vocab_size = 8192;
    int64_t max_seq_len = 512;
    int64_t embed_dim = 768;
    int64_t num_heads = 12;
    int64_t num_layers = 11;
    float calc_eps = 1e-5f;
};

inline int64_t shape_volume(const std::vector<int64_t>& s) {
    int64_t v = 1;
    for (int64_t d : s) v *= d;
    return v;
}
inline std::vector<int64_t> dense_strides(const std::vector<int64_t>& s) {
    std::vector<int64_t> st(s.size());
    int64_t run = 1;
    for (int64_t i = (int64_t)s.size() - 1; i >= 0; --i) { st[i] = run; run *= s[i]; }
    return st;
}

}  // namespace gradc
