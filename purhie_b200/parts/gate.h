// The gate of a gated feed-forward, as the parts and the activation kernel name it.
#pragma once

#include "../host/common.h"
#include "../host/json.h"

namespace qe {

// kind 0: act(g, u) = silu(g) * u.  kind 1 ("clamped_swish"): g' = min(g, limit), u' = clamp(u, -limit, limit),
// act = g' * sigmoid(alpha * g') * (u' + shift).  kind 2 ("gelu_tanh"): act = gelu(g) * u with the tanh form of gelu,
// 0.5 g (1 + tanh(sqrt(2/pi) (g + 0.044715 g^3))).
struct GateSpec {
    int kind = 0;
    float alpha = 1.0f, limit = 0.0f, shift = 0.0f;
    // from a part's params: "activation" absent or null -> silu
    static GateSpec read(const Json& params) {
        GateSpec g;
        const Json* a = params.find("activation");
        if (!a || a->is_null()) return g;
        const std::string kind = a->get_string("kind", "silu");
        if (kind == "silu") return g;
        if (kind == "gelu_tanh") { g.kind = 2; return g; }
        if (kind != "clamped_swish") throw ConfigError("gated feed-forward: activation '" + kind + "' is not known (silu, clamped_swish, gelu_tanh)");
        g.kind = 1;
        g.alpha = (float)a->get_double("alpha", 1.0);
        g.limit = (float)a->at("limit").as_double();
        g.shift = (float)a->get_double("shift", 0.0);
        if (!(g.limit > 0)) throw ConfigError("gated feed-forward: the clamp's limit must be positive");
        return g;
    }
    // what the tensor-core product's epilogue reads on the host: alpha, limit, shift and the kind
    void constants(float out[4]) const { out[0] = alpha; out[1] = limit; out[2] = shift; out[3] = (float)kind; }
};

// An activation of one argument, for a feed-forward without a gate: "silu" (0), "relu2" (1: the square of relu).
inline int unary_activation(const std::string& name) {
    if (name == "silu") return 0;
    if (name == "relu2") return 1;
    throw ConfigError("feed-forward: activation '" + name + "' is not known (silu, relu2)");
}

}  // namespace qe
