// plan.cpp - byte form of the launch plan (see cg/b200/plan.hpp).
#include "cg/b200/plan.hpp"

#include <cstring>

namespace cg::b200 {
namespace {

constexpr std::uint32_t kPlanVersion = 3;

struct Out {
    std::vector<std::uint8_t> bytes;
    template <typename T>
    void put(const T& v) {
        const auto* p = reinterpret_cast<const std::uint8_t*>(&v);
        bytes.insert(bytes.end(), p, p + sizeof(T));
    }
};

struct In {
    const std::vector<std::uint8_t>& bytes;
    std::size_t off = 0;
    bool ok = true;
    template <typename T>
    T get() {
        T v{};
        if (!ok || off + sizeof(T) > bytes.size()) {
            ok = false;
            return v;
        }
        std::memcpy(&v, bytes.data() + off, sizeof(T));
        off += sizeof(T);
        return v;
    }
};

}  // namespace

std::vector<std::uint8_t> LaunchPlan::serialize() const {
    Out o;
    o.put(kMagic);
    o.put(kPlanVersion);
    o.put(static_cast<std::uint32_t>(sizeof(PlanRecord)));
    o.put(n_inputs);
    o.put(n_outputs);
    o.put(workspace_bytes);
    o.put(static_cast<std::uint32_t>(buffers.size()));
    for (const PlanBuffer& b : buffers) {
        o.put(b.bytes);
        o.put(b.dtype);
        o.put(static_cast<std::uint32_t>(b.shape.size()));
        for (std::int64_t d : b.shape) o.put(d);
    }
    o.put(static_cast<std::uint32_t>(records.size()));
    for (const PlanRecord& r : records) o.put(r);
    return o.bytes;
}

std::optional<LaunchPlan> LaunchPlan::deserialize(const std::vector<std::uint8_t>& bytes) {
    In in{bytes};
    LaunchPlan p;
    if (in.get<std::uint32_t>() != kMagic || in.get<std::uint32_t>() != kPlanVersion) return std::nullopt;
    if (in.get<std::uint32_t>() != sizeof(PlanRecord)) return std::nullopt;
    p.n_inputs = in.get<std::uint32_t>();
    p.n_outputs = in.get<std::uint32_t>();
    p.workspace_bytes = in.get<std::uint64_t>();
    const std::uint32_t nb = in.get<std::uint32_t>();
    if (!in.ok || nb > (1u << 20)) return std::nullopt;
    for (std::uint32_t i = 0; i < nb; ++i) {
        PlanBuffer b;
        b.bytes = in.get<std::uint64_t>();
        b.dtype = in.get<std::int32_t>();
        const std::uint32_t rank = in.get<std::uint32_t>();
        if (!in.ok || rank > 16) return std::nullopt;
        for (std::uint32_t k = 0; k < rank; ++k) b.shape.push_back(in.get<std::int64_t>());
        p.buffers.push_back(std::move(b));
    }
    const std::uint32_t nr = in.get<std::uint32_t>();
    if (!in.ok || nr > (1u << 20)) return std::nullopt;
    auto in_range = [&](std::int32_t b) { return b >= -1 && b < static_cast<std::int32_t>(nb); };
    for (std::uint32_t i = 0; i < nr; ++i) {
        PlanRecord r = in.get<PlanRecord>();
        if (!in.ok) return std::nullopt;
        if (r.kind < PlanRecord::Eltwise || r.kind > PlanRecord::Reduce) return std::nullopt;
        for (std::int32_t b : r.input)
            if (!in_range(b)) return std::nullopt;
        for (std::int64_t o : r.input_offset)
            if (o < 0) return std::nullopt;
        if (r.output < 0 || !in_range(r.output) || r.output_offset < 0) return std::nullopt;
        p.records.push_back(r);
    }
    if (!in.ok || in.off != bytes.size() || p.n_inputs + p.n_outputs > nb) return std::nullopt;
    return p;
}

}  // namespace cg::b200
