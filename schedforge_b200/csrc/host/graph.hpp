// Host-side graph layer of the decoder executor: a small Tensor-SSA graph, the line-based
// StableHLO-subset importer, shape inference and the decoder fusion check.  It mirrors
// the part of the reference's graph compiler that sits in front of DecoderCompiler::compile
// (include/schedforge/graph_compiler.h:14-127,363-367; src/graph_compiler.cpp:171-303,
// 1123-1198; src/decoder_compiler.cpp:380-481) with the same names, the same accepted
// text and the same error conditions.
#pragma once

#include <cstdint>
#include <filesystem>
#include <map>
#include <string>
#include <vector>

namespace sfb {

enum class GraphOpKind {
    Input, Constant, MatMul, Add, Multiply, Maximum, Gelu, Broadcast, Reshape, Transpose, Reduce,
    Exp, Rsqrt, Convert, RmsNorm, RoPE, Silu, Concat, Split, FusedQKVProjection,
    FusedGateUpProjection, Softmax, Mask, AttentionSdpa, TopK, MoeHistogram, MoePrefixSum,
    MoeDispatch, MoeGroupedMatMul, SwiGLU, MoeCombine, Return
};

const char* op_name(GraphOpKind kind);

enum class DimensionKind { Static, Dynamic, Symbolic };

struct Dimension {
    DimensionKind kind = DimensionKind::Static;
    std::int64_t value = 1;
    std::string symbol;
    static Dimension fixed(std::int64_t v) { return {DimensionKind::Static, v, {}}; }
    static Dimension dynamic(std::string s = "?") { return {DimensionKind::Dynamic, -1, std::move(s)}; }
    static Dimension symbolic(std::string s) { return {DimensionKind::Symbolic, -1, std::move(s)}; }
    std::string str() const;
    bool matches(const Dimension& other) const;
};

struct GraphTensorType {
    std::vector<Dimension> shape;
    std::string str() const;  // "tensor<4x16xf32, layout=row_major>"
};

struct GraphValue {
    std::string name;
    GraphTensorType type;
    int producer = -1;
    std::vector<int> users;
    bool constant = false;
};

struct GraphOperation {
    GraphOpKind kind = GraphOpKind::Input;
    std::string name;
    std::vector<int> inputs;
    std::vector<int> outputs;
    std::map<std::string, std::string> attributes;
    std::string str(const std::vector<GraphValue>& values) const;
};

class TensorGraph {
public:
    int addInput(std::string name, GraphTensorType type, bool constant = false);
    int addConstant(std::string name, GraphTensorType type, std::string literal);
    int addOperation(GraphOpKind kind, std::string name, std::vector<int> inputs, GraphTensorType type = {});
    void setReturn(int value);
    int returnValue() const { return return_value_; }
    std::vector<GraphValue>& values() { return values_; }
    const std::vector<GraphValue>& values() const { return values_; }
    std::vector<GraphOperation>& operations() { return operations_; }
    const std::vector<GraphOperation>& operations() const { return operations_; }
    std::string dump() const;
private:
    std::vector<GraphValue> values_;
    std::vector<GraphOperation> operations_;
    int return_value_ = -1;
};

struct ShapeConstraint {
    std::string expression;
    bool runtime_guard = false;
};

class ShapeInferencePass {
public:
    std::vector<ShapeConstraint> run(TensorGraph& graph) const;  // throws std::invalid_argument
};

class StableHLOImporter {
public:
    TensorGraph importFile(const std::filesystem::path& path) const;  // std::runtime_error if unreadable
    TensorGraph importText(const std::string& text) const;            // std::invalid_argument on bad input
};

enum class DecoderFFNKind { Dense, MoE };

struct DecoderFusionSummary {
    bool fused_qkv = false;
    bool fused_gate_up = false;
    bool fused_rope = false;
    std::string dump() const;
};

class DecoderFusionPass {
public:
    DecoderFusionSummary run(const TensorGraph& graph, DecoderFFNKind ffn) const;
};

}  // namespace sfb
