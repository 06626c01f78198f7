#include "graph.hpp"

#include <algorithm>
#include <fstream>
#include <iterator>
#include <regex>
#include <sstream>
#include <stdexcept>
#include <unordered_map>

namespace sfb {

const char* op_name(GraphOpKind kind) {
    static const char* const names[] = {
        "tensor.input", "tensor.constant", "tensor.matmul", "tensor.add", "tensor.multiply",
        "tensor.maximum", "tensor.gelu", "tensor.broadcast", "tensor.reshape", "tensor.transpose",
        "tensor.reduce", "tensor.exp", "tensor.rsqrt", "tensor.convert", "tensor.rms_norm",
        "tensor.rope", "tensor.silu", "tensor.concat", "tensor.split", "tensor.fused_qkv",
        "tensor.fused_gate_up", "tensor.softmax", "tensor.mask", "attention.sdpa", "tensor.topk",
        "moe.histogram", "moe.prefix_sum", "moe.dispatch", "moe.grouped_matmul", "tensor.swiglu",
        "moe.combine", "func.return"};
    const auto index = static_cast<std::size_t>(kind);
    return index < std::size(names) ? names[index] : "tensor.unknown";
}

std::string Dimension::str() const {
    if (kind == DimensionKind::Static) return std::to_string(value);
    return symbol.empty() ? "?" : symbol;
}

bool Dimension::matches(const Dimension& other) const {
    if (kind == DimensionKind::Static && other.kind == DimensionKind::Static) return value == other.value;
    return kind == DimensionKind::Dynamic || other.kind == DimensionKind::Dynamic || str() == other.str();
}

std::string GraphTensorType::str() const {
    std::string text = "tensor<";
    for (const auto& d : shape) text += d.str() + "x";
    return text + "f32, layout=row_major>";
}

std::string GraphOperation::str(const std::vector<GraphValue>& values) const {
    std::ostringstream out;
    if (!outputs.empty()) out << "%v" << outputs.front() << " = ";
    out << op_name(kind);
    for (const int input : inputs) out << " %v" << input;
    if (!attributes.empty()) {
        out << " {";
        bool first = true;
        for (const auto& [key, value] : attributes) {  // std::map iterates in key order
            out << (first ? "" : ", ") << key << '=' << value;
            first = false;
        }
        out << '}';
    }
    if (!outputs.empty()) out << " : " << values.at(static_cast<std::size_t>(outputs.front())).type.str();
    return out.str();
}

int TensorGraph::addInput(std::string name, GraphTensorType type, bool constant) {
    const int value = static_cast<int>(values_.size());
    const int op = static_cast<int>(operations_.size());
    operations_.push_back({constant ? GraphOpKind::Constant : GraphOpKind::Input, name, {}, {value}, {}});
    values_.push_back({std::move(name), std::move(type), op, {}, constant});
    return value;
}

int TensorGraph::addConstant(std::string name, GraphTensorType type, std::string literal) {
    const int value = addInput(std::move(name), std::move(type), true);
    operations_.back().attributes["value"] = std::move(literal);
    return value;
}

int TensorGraph::addOperation(GraphOpKind kind, std::string name, std::vector<int> inputs, GraphTensorType type) {
    const int value = static_cast<int>(values_.size());
    const int op = static_cast<int>(operations_.size());
    for (const int input : inputs) values_.at(static_cast<std::size_t>(input)).users.push_back(op);
    values_.push_back({name + ".result", std::move(type), op, {}, false});
    operations_.push_back({kind, std::move(name), std::move(inputs), {value}, {}});
    return value;
}

void TensorGraph::setReturn(int value) {
    values_.at(static_cast<std::size_t>(value)).users.push_back(static_cast<int>(operations_.size()));
    operations_.push_back({GraphOpKind::Return, "return", {value}, {}, {}});
    return_value_ = value;
}

std::string TensorGraph::dump() const {
    std::string text = "graph @model {\n";
    for (const auto& op : operations_) text += "  " + op.str(values_) + "\n";
    return text + "}\n";
}

std::vector<ShapeConstraint> ShapeInferencePass::run(TensorGraph& graph) const {
    std::vector<ShapeConstraint> constraints;
    for (const auto& value : graph.values())
        for (const auto& d : value.type.shape)
            if (d.kind != DimensionKind::Static) constraints.push_back({d.str() + " > 0", true});
    auto type_of = [&](int value) -> const GraphTensorType& {
        return graph.values().at(static_cast<std::size_t>(value)).type;
    };
    auto dynamic_pair = [](const Dimension& a, const Dimension& b) {
        return a.kind != DimensionKind::Static || b.kind != DimensionKind::Static;
    };
    for (auto& op : graph.operations()) {
        if (op.outputs.empty()) continue;
        GraphTensorType& out = graph.values().at(static_cast<std::size_t>(op.outputs[0])).type;
        switch (op.kind) {
            case GraphOpKind::MatMul: {
                const auto lhs = type_of(op.inputs.at(0)), rhs = type_of(op.inputs.at(1));
                if (lhs.shape.size() == 2 && rhs.shape.size() == 2) {
                    if (!lhs.shape[1].matches(rhs.shape[0]))
                        throw std::invalid_argument("matmul reduction dimensions do not match");
                    constraints.push_back({lhs.shape[1].str() + " == " + rhs.shape[0].str(),
                                           dynamic_pair(lhs.shape[1], rhs.shape[0])});
                    out.shape = {lhs.shape[0], rhs.shape[1]};
                } else if (lhs.shape.size() == 4 && rhs.shape.size() == 4) {
                    if (!lhs.shape[0].matches(rhs.shape[0]) || !lhs.shape[3].matches(rhs.shape[2]))
                        throw std::invalid_argument("batched matmul dimensions do not match");
                    if (!dynamic_pair(lhs.shape[1], rhs.shape[1]) && lhs.shape[1].value % rhs.shape[1].value != 0)
                        throw std::invalid_argument("batched matmul head dimensions do not broadcast");
                    constraints.push_back({lhs.shape[3].str() + " == " + rhs.shape[2].str(),
                                           dynamic_pair(lhs.shape[3], rhs.shape[2])});
                    constraints.push_back({lhs.shape[1].str() + " % " + rhs.shape[1].str() + " == 0",
                                           dynamic_pair(lhs.shape[1], rhs.shape[1])});
                    out.shape = {lhs.shape[0], lhs.shape[1], lhs.shape[2], rhs.shape[3]};
                } else {
                    throw std::invalid_argument("matmul requires matching rank-2 or rank-4 tensors");
                }
                break;
            }
            case GraphOpKind::Add:
            case GraphOpKind::Multiply:
            case GraphOpKind::Maximum: {
                const auto lhs = type_of(op.inputs.at(0)), rhs = type_of(op.inputs.at(1));
                out = lhs.shape.size() >= rhs.shape.size() ? lhs : rhs;
                break;
            }
            case GraphOpKind::RmsNorm:
            case GraphOpKind::RoPE:
            case GraphOpKind::Silu:
                out = type_of(op.inputs.at(0));
                break;
            case GraphOpKind::FusedQKVProjection:
            case GraphOpKind::FusedGateUpProjection: {
                const auto lhs = type_of(op.inputs.at(0)), rhs = type_of(op.inputs.at(1));
                if (lhs.shape.size() != 2 || rhs.shape.size() != 2 || !lhs.shape[1].matches(rhs.shape[0]))
                    throw std::invalid_argument("fused projection requires compatible rank-2 tensors");
                out.shape = {lhs.shape[0], rhs.shape[1]};
                break;
            }
            case GraphOpKind::Concat:
            case GraphOpKind::Split:
                if (op.inputs.empty()) throw std::invalid_argument("concat/split requires input");
                if (out.shape.empty()) out = type_of(op.inputs[0]);
                break;
            case GraphOpKind::AttentionSdpa: {
                const auto q = type_of(op.inputs.at(0)), k = type_of(op.inputs.at(1)), v = type_of(op.inputs.at(2));
                if (q.shape.size() != 4 || k.shape.size() != 4 || v.shape.size() != 4)
                    throw std::invalid_argument("attention.sdpa requires rank-4 Q/K/V tensors");
                if (!q.shape[0].matches(k.shape[0]) || !k.shape[0].matches(v.shape[0]) ||
                    !q.shape[3].matches(k.shape[3]) || !k.shape[2].matches(v.shape[2]))
                    throw std::invalid_argument("attention.sdpa Q/K/V dimensions do not match");
                out.shape = {q.shape[0], q.shape[1], q.shape[2], v.shape[3]};
                constraints.push_back({q.shape[1].str() + " % " + k.shape[1].str() + " == 0",
                                       dynamic_pair(q.shape[1], k.shape[1])});
                break;
            }
            case GraphOpKind::Gelu: case GraphOpKind::Exp: case GraphOpKind::Rsqrt:
            case GraphOpKind::Convert: case GraphOpKind::Broadcast: case GraphOpKind::Softmax:
            case GraphOpKind::Mask: case GraphOpKind::SwiGLU: case GraphOpKind::MoeCombine:
                if (out.shape.empty() && !op.inputs.empty()) out = type_of(op.inputs[0]);
                break;
            default:
                break;
        }
    }
    return constraints;
}

namespace {

GraphTensorType parse_tensor_type(const std::string& text) {
    const auto begin = text.find("tensor<");
    const auto end = begin == std::string::npos ? std::string::npos : text.find('>', begin);
    if (begin == std::string::npos || end == std::string::npos)
        throw std::invalid_argument("missing tensor type: " + text);
    std::string body = text.substr(begin + 7, end - begin - 7);
    if (body.size() >= 4 && body.compare(body.size() - 4, 4, "xf32") == 0) body.resize(body.size() - 4);
    GraphTensorType type;
    std::stringstream stream(body);
    std::string extent;
    while (std::getline(stream, extent, 'x')) {
        if (extent.empty()) continue;
        if (extent == "?") type.shape.push_back(Dimension::dynamic());
        else if (std::all_of(extent.begin(), extent.end(), [](unsigned char c) { return std::isdigit(c) != 0; }))
            type.shape.push_back(Dimension::fixed(std::stoll(extent)));
        else type.shape.push_back(Dimension::symbolic(extent));
    }
    return type;
}

bool classify(const std::string& op, const std::string& operands, GraphOpKind& kind) {
    static const std::unordered_map<std::string, GraphOpKind> plain = {
        {"constant", GraphOpKind::Constant}, {"dot_general", GraphOpKind::MatMul}, {"dot", GraphOpKind::MatMul},
        {"add", GraphOpKind::Add}, {"multiply", GraphOpKind::Multiply}, {"maximum", GraphOpKind::Maximum},
        {"broadcast_in_dim", GraphOpKind::Broadcast}, {"reshape", GraphOpKind::Reshape},
        {"transpose", GraphOpKind::Transpose}, {"reduce", GraphOpKind::Reduce},
        {"exponential", GraphOpKind::Exp}, {"rsqrt", GraphOpKind::Rsqrt}, {"convert", GraphOpKind::Convert}};
    if (const auto found = plain.find(op); found != plain.end()) { kind = found->second; return true; }
    if (op != "custom_call") return false;
    static const std::pair<const char*, GraphOpKind> calls[] = {
        {"RmsNorm", GraphOpKind::RmsNorm}, {"RoPE", GraphOpKind::RoPE}, {"SwiGLU", GraphOpKind::SwiGLU},
        {"SiLU", GraphOpKind::Silu}, {"MoeFFN", GraphOpKind::MoeCombine}, {"Gelu", GraphOpKind::Gelu}};
    for (const auto& [target, mapped] : calls)
        if (operands.find(target) != std::string::npos) { kind = mapped; return true; }
    return false;
}

}  // namespace

TensorGraph StableHLOImporter::importFile(const std::filesystem::path& path) const {
    std::ifstream input(path);
    if (!input) throw std::runtime_error("cannot open StableHLO file: " + path.string());
    return importText(std::string(std::istreambuf_iterator<char>(input), std::istreambuf_iterator<char>()));
}

TensorGraph StableHLOImporter::importText(const std::string& text) const {
    static const std::regex argument(R"((%[A-Za-z0-9_]+)\s*:\s*(tensor<[^>]+>))");
    static const std::regex assignment(
        R"((%[A-Za-z0-9_]+)\s*=\s*stablehlo\.([A-Za-z0-9_]+)\s+([^:]+)(?::\s*(tensor<[^>]+>))?)");
    static const std::regex ssa_name(R"(%[A-Za-z0-9_]+)");
    TensorGraph graph;
    std::unordered_map<std::string, int> known;
    std::istringstream lines(text);
    for (std::string line; std::getline(lines, line);) {
        for (std::sregex_iterator it(line.begin(), line.end(), argument), end; it != end; ++it) {
            const std::string name = (*it)[1];
            if (!known.count(name)) known[name] = graph.addInput(name.substr(1), parse_tensor_type((*it)[2]));
        }
        const bool has_op = line.find("stablehlo.") != std::string::npos;
        if (line.find("func.func") != std::string::npos || (line.find('=') == std::string::npos && !has_op))
            continue;
        std::smatch match;
        if (std::regex_search(line, match, assignment)) {
            const std::string result = match[1], op = match[2], operand_text = match[3];
            std::vector<int> operands;
            for (std::sregex_iterator it(operand_text.begin(), operand_text.end(), ssa_name), end; it != end; ++it)
                if (const auto found = known.find(it->str()); found != known.end()) operands.push_back(found->second);
            GraphOpKind kind;
            if (!classify(op, operand_text, kind))
                throw std::invalid_argument("unsupported StableHLO operation: " + op);
            GraphTensorType type;
            if (match[4].matched) type = parse_tensor_type(match[4]);
            known[result] = kind == GraphOpKind::Constant
                ? graph.addConstant(result.substr(1), std::move(type), operand_text)
                : graph.addOperation(kind, result.substr(1), std::move(operands), std::move(type));
        } else if (line.find("return") != std::string::npos) {
            std::smatch returned;
            if (std::regex_search(line, returned, ssa_name) && known.count(returned.str()))
                graph.setReturn(known[returned.str()]);
        }
    }
    if (graph.returnValue() < 0 && !graph.values().empty())
        graph.setReturn(static_cast<int>(graph.values().size()) - 1);
    ShapeInferencePass{}.run(graph);
    return graph;
}

std::string DecoderFusionSummary::dump() const {
    return "decoder.fusion qkv=" + std::to_string(fused_qkv) + " gate_up=" + std::to_string(fused_gate_up) +
           " rope=" + std::to_string(fused_rope);
}

DecoderFusionSummary DecoderFusionPass::run(const TensorGraph& graph, DecoderFFNKind) const {
    DecoderFusionSummary summary;
    std::unordered_map<int, int> matmul_fanout;  // value -> MatMuls that read it as input 0
    const auto& ops = graph.operations();
    const auto& values = graph.values();
    auto producer_of = [&](int value) -> const GraphOperation* {
        const int p = values.at(static_cast<std::size_t>(value)).producer;
        return p >= 0 ? &ops.at(static_cast<std::size_t>(p)) : nullptr;
    };
    for (const auto& op : ops) {
        if (op.kind == GraphOpKind::MatMul && !op.inputs.empty()) ++matmul_fanout[op.inputs.front()];
        if (op.kind == GraphOpKind::RoPE || op.name.find("rope") != std::string::npos) summary.fused_rope = true;
        if (op.kind == GraphOpKind::FusedQKVProjection) summary.fused_qkv = true;
        if (op.kind == GraphOpKind::SwiGLU && op.inputs.size() >= 2) {
            const GraphOperation* gate = producer_of(op.inputs[0]);
            const GraphOperation* up = producer_of(op.inputs[1]);
            // As in the reference, the last SwiGLU seen decides the pattern flag.
            if (gate && up)
                summary.fused_gate_up = gate->kind == GraphOpKind::MatMul && up->kind == GraphOpKind::MatMul &&
                    !gate->inputs.empty() && !up->inputs.empty() && gate->inputs.front() == up->inputs.front();
        }
    }
    for (const auto& [value, count] : matmul_fanout)
        if (count >= 3) summary.fused_qkv = true;
    for (const auto& op : ops)
        if (op.kind == GraphOpKind::FusedGateUpProjection) summary.fused_gate_up = true;
    return summary;
}

}  // namespace sfb
