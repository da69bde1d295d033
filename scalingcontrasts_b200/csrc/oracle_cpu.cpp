// Float64 evaluation of the one-set Matryoshka sigmoid loss as plain loops over ordered pairs: the cross-check of the
// vectorised Python oracle. Each ordered cell adds its gradient to both of its rows, which is where the factor two of
// the row-owned kernels comes from. Parity: oracle_loss (scalingcontrasts.cu:133-170), extended with the pair-positive
// and diagonal options.
#include <cmath>
#include <vector>

#include "api.h"

namespace sc {

void oracle_loops_f64(double const* world, size_t n, size_t hidden, ladder_host const& ladder, double beta, double bias,
                      uint32_t spec_code, double* gradient, double* out) {
    bool const pairs = (spec_code & 1u) != 0u;
    uint32_t const diagonal_rule = (spec_code >> 1) & 3u;
    double const weight = 1.0 / static_cast<double>(n);
    for (size_t i = 0; i < n * hidden; ++i) gradient[i] = 0.0;
    for (int i = 0; i < 12; ++i) out[i] = 0.0;
    std::vector<double> norms(n);
    for (uint32_t band = 0; band < ladder.count; ++band) {
        size_t const width = ladder.ends[band];
        for (size_t i = 0; i < n; ++i) {
            double sum = 0;
            for (size_t h = 0; h < width; ++h) sum += world[i * hidden + h] * world[i * hidden + h];
            norms[i] = std::sqrt(sum);
        }
        for (size_t i = 0; i < n; ++i)
            for (size_t j = 0; j < n; ++j) {
                bool const diagonal = i == j;
                if (diagonal && diagonal_rule == 2u) continue;
                double dot = 0;
                for (size_t h = 0; h < width; ++h) dot += world[i * hidden + h] * world[j * hidden + h];
                double const denominator = norms[i] * norms[j];
                bool const active = denominator > 1e-2;
                double const cosine = diagonal ? 1.0 : (active ? dot / denominator : 0.0);
                double target = -1.0;
                if (pairs && (i ^ 1) == j) target = 1.0;
                if (diagonal && diagonal_rule == 0u) target = 1.0;
                double const logit = beta * cosine;
                double const s = target * (logit + bias);
                double const cell_loss = weight * (std::fmax(-s, 0.0) + std::log1p(std::exp(-std::fabs(s))));
                out[0] += cell_loss;
                out[4 + band] += cell_loss;
                double const cell_grad = -weight * target / (1.0 + std::exp(s));
                out[1] += cell_grad;
                out[2] += cell_grad * logit;
                if (diagonal || !active) continue;
                double const scaled = cell_grad * beta;
                for (size_t h = 0; h < width; ++h) {
                    double const vi = world[i * hidden + h], vj = world[j * hidden + h];
                    gradient[i * hidden + h] += scaled * (vj / denominator - cosine * vi / (norms[i] * norms[i]));
                    gradient[j * hidden + h] += scaled * (vi / denominator - cosine * vj / (norms[j] * norms[j]));
                }
            }
    }
}

} // namespace sc
