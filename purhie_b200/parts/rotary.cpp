// Rotary position encoding, rotate-half pairing.
//
// For pair i < n_rot/2 the angle at position p is p * theta^(-2i/n_rot) (times an optional per-pair frequency
// factor); (x_i, x_{i+n_rot/2}) turns by it; dimensions >= n_rot are left alone.  Angles are computed in double
// precision on the host and stored as float32 cosines and sines.  Reference: src/qwen_ops.cpp:15-24 (double
// theta), src/attention.hip:225-240 (the device version); base and width: src/inference.cpp:1358-1359; the
// frequency factors and the interleaved pairing are the reference's knobs of src/attention.h:69, 84-95.
#include <cmath>

#include "parts.h"

namespace qe {

// params: theta, n_rot, max_position; optional pairing ("half" | "interleaved"), freq_factors [n_rot/2] (each
// pair's frequency is divided by its factor), position_column.
class RotaryTable : public PositionEncoding {
public:
    RotaryTable(const Json& p, BuildContext& b) : PositionEncoding(p, b) {
        theta_ = p.at("theta").as_double();
        n_rot_ = (int)p.at("n_rot").as_int();
        max_position_ = p.at("max_position").as_int();
        interleaved_ = p.get_string("pairing", "half") == "interleaved";
        column_ = (int)p.get_int("position_column", 0);
        if (n_rot_ % 2 || n_rot_ < 2) throw ConfigError("rotary width " + std::to_string(n_rot_) + " must be even and at least 2");
        if (!(theta_ > 0) || max_position_ < 1) throw ConfigError("rotary: theta must be positive and max_position at least 1");
        if (const Json* f = p.find("freq_factors")) {
            if (!f->is_null()) {
                if (!f->is_array() || (int)f->size() != n_rot_ / 2) throw ConfigError("rotary: freq_factors must list n_rot/2 numbers");
                for (const Json& v : f->items()) factors_.push_back(v.as_double());
            }
        }
    }
    int n_rot() const override { return n_rot_; }
    bool interleaved() const override { return interleaved_; }
    int position_column() const override { return column_; }

    void bind(WeightSource& src) override {
        if (table_.defined()) return;                     // shared by all layers: made once
        const int half = n_rot_ / 2;
        std::vector<float> host((size_t)max_position_ * n_rot_);
        std::vector<double> inv(half);
        for (int i = 0; i < half; i++) {
            inv[i] = std::pow(theta_, -2.0 * i / n_rot_);
            if (!factors_.empty()) inv[i] /= factors_[i];
        }
        for (int64_t pos = 0; pos < max_position_; pos++)
            for (int i = 0; i < half; i++) {
                const double a = (double)pos * inv[i];
                host[(size_t)pos * n_rot_ + i] = (float)std::cos(a);
                host[(size_t)pos * n_rot_ + half + i] = (float)std::sin(a);
            }
        table_ = src.arena().alloc(DType::F32, {max_position_, n_rot_});
        QE_CUDA(cudaMemcpy(table_.data, host.data(), host.size() * sizeof(float), cudaMemcpyHostToDevice));
    }
    Tensor rotation_table() override { return table_; }

private:
    double theta_;
    int n_rot_, column_;
    int64_t max_position_;
    bool interleaved_;
    std::vector<double> factors_;
    Tensor table_;
};

void register_position_parts() {
    register_part("position", "rope_neox", [](const Json& p, BuildContext& b) { return std::make_shared<RotaryTable>(p, b); });
}

}  // namespace qe
