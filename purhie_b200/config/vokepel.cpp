// The Vokepel design: a pre-norm decoder with a factor on everything a part adds, whose mixers are either attention with
// heads that talk to each other before the softmax, or grouped-query attention with a sink side by side with a minimal
// gated recurrent unit, and of which a stretch of layers may run several times in a row with the same weights.
//
//     e = embed[token]
//     a layer:  x <- x + m * mixer(rms(x; norm1));  x <- x + m * ff(rms(x; norm2))            m = residual_mult
//     before pass t of the stretch [loop.start, loop.stop):  x <- W_in [x ; e] + step[t]
//     logits = cap * tanh(embed rms(x; final.norm) * logit_scale / cap)                     the head is the embedding table
//   mixer "attention": q and k RMS-normed over the whole projection, the values are the keys as projected; scores times
//     `scale`, capped (softcap * tanh(s / softcap)), minus r1_h ln(1 + r2_h * distance), mixed across heads by `talk`,
//     softmax over the last mask.size positions; the heads times sigmoid(W_g h); W_o.
//   mixer "parallel": left_scale * left + right_scale * right; left is grouped-query attention with interleaved rotary
//     pairs on the first rot.dims dimensions of a head, a window and a sink in the softmax; right is the recurrent unit
//     of parts/min_gru.cpp.
//   feed-forward "dense": W_down relu(W_up h)^2.
//
// config.json keys, all read here and nowhere else:
//   architecture ("Vokepel"), vocab, width, norm.eps, residual_mult (default 1), logit_scale (default 1), logit_softcap
//   (optional), layers[i].type ("attention" | "parallel"), layers[i].mixer, layers[i].mlp (null: no feed-forward; kind
//   "dense": ff), loop {start, stop, times} (optional);
//   an attention mixer or the left side: heads, kv_heads, dim, vdim, scale, mask {size} (optional: every earlier position
//     is seen); the attention mixer also softcap (optional); the left side also rot {base, dims} (optional);
//   a parallel mixer: left {...}, right {width}, left_scale, right_scale;
//   max_position (optional): the longest sequence the rotary table is made for.
// Tensor names: embed, final.norm, loop.in, loop.step, and per layer i: l<i>.norm1, l<i>.norm2,
// l<i>.mix.{q, k, q.norm, k.norm, r1, r2, talk, g, o} or l<i>.mix.left.{q, k, v, sink, o} and
// l<i>.mix.right.{z, z.b, x, x.b, g, o}; l<i>.mlp.{up, down}.
//
// What the design fixes and the code therefore states: the norms are RMS norms with plain weights; the feed-forward's
// activation is the square of relu; rotary pairs are (2i, 2i + 1); the values of an attention mixer are its keys before
// their norm; the gate of that mixer is a sigmoid.
#include "config.h"

namespace qe {

namespace {
constexpr long long kDefaultMaxPosition = 65536;
const char* const kActivation = "relu2";

Json names(std::initializer_list<std::pair<const char*, std::string>> list) {
    Json n = Json::object();
    for (const auto& kv : list) n.set(kv.first, kv.second);
    return n;
}
const Json& object_at(const Json& d, const std::string& key, const std::string& where) {
    const Json* v = d.find(key);
    if (!v || !v->is_object()) throw ConfigError("config.json: " + where + "'" + key + "' must be an object");
    return *v;
}
// heads, kv_heads, dim, vdim, scale, mask of an attention mixer (the talking one or the left side of a pair)
void check_attention(const Json& m, const std::string& where) {
    const long long heads = take_int(m, "heads"), kv = take_int(m, "kv_heads");
    take_int(m, "dim"); take_int(m, "vdim");
    if (heads % kv) throw ConfigError("config.json: " + where + "heads " + std::to_string(heads) + " is no multiple of kv_heads " + std::to_string(kv));
    if (!(take_float(m, "scale") > 0.0)) throw ConfigError("config.json: " + where + "scale must be positive");
    if (has_value(m, "mask")) take_int(object_at(m, "mask", where), "size");
}
}  // namespace

class VokepelConfig : public ModelConfig {
public:
    Json source;                        // config.json as read (checked)
    long long vocab = 0, width = 0, max_position = kDefaultMaxPosition;
    long long loop_start = 0, loop_stop = 0, loop_times = 0;        // times 0: no stretch is repeated
    double eps = 0.0, residual_mult = 1.0, logit_scale = 1.0, logit_softcap = 0.0;

    static std::unique_ptr<ModelConfig> read(const Json& d) {
        std::unique_ptr<VokepelConfig> c(new VokepelConfig());
        c->architecture = "Vokepel";
        c->source = d;
        c->vocab = take_int(d, "vocab");
        c->width = take_int(d, "width");
        c->eps = take_float(object_at(d, "norm", ""), "eps");
        if (!(c->eps > 0.0)) throw ConfigError("config.json: norm.eps must be positive");
        c->residual_mult = take_float(d, "residual_mult", 1.0);
        c->logit_scale = take_float(d, "logit_scale", 1.0);
        c->logit_softcap = has_value(d, "logit_softcap") ? take_float(d, "logit_softcap") : 0.0;
        if (c->logit_softcap < 0.0) throw ConfigError("config.json: logit_softcap must be positive");
        c->max_position = take_int(d, "max_position", kDefaultMaxPosition, 1);
        const Json* layers = d.find("layers");
        if (!layers || !layers->is_array() || layers->size() == 0) throw ConfigError("config.json: 'layers' must be a non-empty list");
        for (size_t i = 0; i < layers->size(); i++) {
            const Json& l = (*layers)[i];
            const std::string where = "layers[" + std::to_string(i) + "].";
            if (!l.is_object()) throw ConfigError("config.json: " + where + " must be an object");
            const std::string type = l.get_string("type", "");
            const Json& m = object_at(l, "mixer", where);
            if (type == "attention") {
                check_attention(m, where + "mixer.");
                if (take_int(m, "vdim") != take_int(m, "dim"))
                    throw ConfigError("config.json: " + where + "mixer: the values are the keys, so vdim must equal dim");
                if (has_value(m, "softcap") && !(take_float(m, "softcap") > 0.0)) throw ConfigError("config.json: " + where + "mixer.softcap must be positive");
            } else if (type == "parallel") {
                const Json& left = object_at(m, "left", where + "mixer.");
                check_attention(left, where + "mixer.left.");
                if (has_value(left, "rot")) {
                    const Json& rot = object_at(left, "rot", where + "mixer.left.");
                    const long long dims = take_int(rot, "dims", 2);
                    if (dims % 2 || dims > take_int(left, "dim")) throw ConfigError("config.json: " + where + "mixer.left.rot.dims must be even and at most dim");
                    if (!(take_float(rot, "base") > 0.0)) throw ConfigError("config.json: " + where + "mixer.left.rot.base must be positive");
                }
                take_int(object_at(m, "right", where + "mixer."), "width");
                take_float(m, "left_scale"); take_float(m, "right_scale");
            } else {
                throw ConfigError("config.json: " + where + "type '" + type + "' is not known (attention, parallel)");
            }
            if (has_value(l, "mlp")) {
                const Json& f = object_at(l, "mlp", where);
                const std::string kind = f.get_string("kind", "");
                if (kind != "dense") throw ConfigError("config.json: " + where + "mlp.kind '" + kind + "' is not known (dense)");
                take_int(f, "ff");
            }
        }
        if (has_value(d, "loop")) {
            const Json& loop = object_at(d, "loop", "");
            c->loop_start = take_int(loop, "start", 0);
            c->loop_stop = take_int(loop, "stop", 0);
            c->loop_times = take_int(loop, "times", 1);
            if (c->loop_start >= c->loop_stop || c->loop_stop > (long long)layers->size())
                throw ConfigError("config.json: loop: layers " + std::to_string(c->loop_start) + " .. " + std::to_string(c->loop_stop) +
                                  " - 1 are no stretch of the " + std::to_string(layers->size()) + " layers");
        }
        return std::unique_ptr<ModelConfig>(c.release());
    }

    Json to_json() const override {
        Json d = source;
        d.set("architecture", "Vokepel");
        return d;
    }

    ModelSpec build_spec() const override {
        auto norm = [&](const std::string& name) {
            Json p = Json::object();
            p.set("size", width);
            p.set("eps", eps);
            p.set("names", names({{"weight", name}}));
            return PartSpec("rmsnorm", p);
        };
        auto window_of = [&](const Json& m) { return has_value(m, "mask") ? m.at("mask").at("size") : Json(0); };
        ModelSpec spec;
        spec.hidden_size = width;
        spec.vocab_size = vocab;
        spec.max_position = max_position;
        const Json& layers = source.at("layers");
        for (size_t i = 0; i < layers.size(); i++) {
            const Json& l = layers[i];
            const Json& m = l.at("mixer");
            const std::string p = "l" + std::to_string(i) + ".";
            const std::string mp = p + "mix.";
            LayerSpec layer;
            layer.arrangement = "pre_norm";
            layer.params.set("residual_factor", residual_mult);
            layer.parts.push_back({"mixer_norm", norm(p + "norm1")});
            if (l.at("type").as_string() == "attention") {
                Json a = Json::object();
                a.set("hidden_size", width);
                a.set("num_heads", m.at("heads"));
                a.set("num_kv_heads", m.at("kv_heads"));
                a.set("head_dim", m.at("dim"));
                a.set("value_dim", m.at("vdim"));
                a.set("values", "keys");
                a.set("joint_norm_eps", eps);
                a.set("window", window_of(m));
                a.set("scale", m.at("scale"));
                a.set("softcap", has_value(m, "softcap") ? m.at("softcap") : Json());
                a.set("names", names({{"q_proj", mp + "q"}, {"k_proj", mp + "k"}, {"o_proj", mp + "o"}, {"q_norm", mp + "q.norm"}, {"k_norm", mp + "k.norm"},
                                      {"distance_slope", mp + "r1"}, {"distance_rate", mp + "r2"}, {"head_mix", mp + "talk"}, {"gate_proj", mp + "g"}}));
                layer.parts.push_back({"mixer", PartSpec("talking_attention", a)});
            } else {
                const Json& lm = m.at("left");
                const std::string lp = mp + "left.", rp = mp + "right.";
                Json a = Json::object();
                a.set("hidden_size", width);
                a.set("num_heads", lm.at("heads"));
                a.set("num_kv_heads", lm.at("kv_heads"));
                a.set("head_dim", lm.at("dim"));
                a.set("value_dim", lm.at("vdim"));
                a.set("qk_norm_eps", Json());
                a.set("bias", false);
                a.set("window", window_of(lm));
                a.set("scale", lm.at("scale"));
                if (has_value(lm, "rot")) {
                    const Json& rot = lm.at("rot");
                    Json pos = Json::object();
                    pos.set("theta", rot.at("base"));
                    pos.set("n_rot", rot.at("dims"));
                    pos.set("max_position", max_position);
                    pos.set("pairing", "interleaved");
                    a.set("position", PartSpec("rope_neox", pos).to_json());
                } else {
                    a.set("position", Json());
                }
                a.set("names", names({{"q_proj", lp + "q"}, {"k_proj", lp + "k"}, {"v_proj", lp + "v"}, {"o_proj", lp + "o"}, {"sink", lp + "sink"}}));
                Json r = Json::object();
                r.set("hidden_size", width);
                r.set("width", m.at("right").at("width"));
                r.set("names", names({{"z_proj", rp + "z"}, {"z_bias", rp + "z.b"}, {"x_proj", rp + "x"}, {"x_bias", rp + "x.b"}, {"g_proj", rp + "g"},
                                      {"o_proj", rp + "o"}}));
                Json pair = Json::object();
                pair.set("hidden_size", width);
                pair.set("combine", "weighted_sum");
                pair.set("left_factor", m.at("left_scale"));
                pair.set("right_factor", m.at("right_scale"));
                pair.set("left", PartSpec("attention", a).to_json());
                pair.set("right", PartSpec("min_gru", r).to_json());
                layer.parts.push_back({"mixer", PartSpec("side_by_side", pair)});
            }
            if (has_value(l, "mlp")) {
                const Json& f = l.at("mlp");
                Json g = Json::object();
                g.set("hidden_size", width);
                g.set("intermediate_size", f.at("ff"));
                g.set("activation", kActivation);
                g.set("names", names({{"up_proj", p + "mlp.up"}, {"down_proj", p + "mlp.down"}}));
                layer.parts.push_back({"feed_forward_norm", norm(p + "norm2")});
                layer.parts.push_back({"feed_forward", PartSpec("mlp", g)});
            }
            spec.layers.push_back(std::move(layer));
        }
        // the run order: the stretch [start, stop) `times` times in a row, a reinjection in front of every round, each
        // round with cache entries of its own
        const int n = (int)layers.size();
        if (loop_times > 0) {
            LayerSpec again;
            again.arrangement = "reinject";
            again.params.set("hidden_size", width);
            again.params.set("passes", loop_times);
            again.params.set("names", names({{"weight", "loop.in"}, {"step", "loop.step"}}));
            spec.layers.push_back(std::move(again));
            spec.keep_embedding_output = true;
            for (int i = 0; i < (int)loop_start; i++) spec.schedule.push_back(LayerCall{i, -1, 0});
            for (int t = 0; t < (int)loop_times; t++) {
                spec.schedule.push_back(LayerCall{n, -1, t});
                for (int i = (int)loop_start; i < (int)loop_stop; i++) spec.schedule.push_back(LayerCall{i, -1, t});
            }
            for (int i = (int)loop_stop; i < n; i++) spec.schedule.push_back(LayerCall{i, -1, 0});
        } else {
            for (int i = 0; i < n; i++) spec.schedule.push_back(LayerCall{i, -1, 0});
        }
        Json e = Json::object();
        e.set("vocab_size", vocab);
        e.set("hidden_size", width);
        e.set("names", names({{"weight", "embed"}}));
        spec.embedding = PartSpec("embedding", e);
        Json h = Json::object();
        h.set("hidden_size", width);
        h.set("vocab_size", vocab);
        h.set("tied_to", "embed");
        h.set("scale", logit_scale);
        h.set("softcap", logit_softcap > 0.0 ? Json(logit_softcap) : Json());
        spec.head = PartSpec("lm_head", h);
        spec.final_norm = norm("final.norm");
        spec.validate();
        return spec;
    }
};

void register_vokepel_architecture() { register_architecture("Vokepel", VokepelConfig::read); }

}  // namespace qe
