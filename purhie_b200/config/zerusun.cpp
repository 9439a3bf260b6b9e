// The Zerusun design: a decoder whose layers have one norm that both of their parts read, whose norm is a dynamic
// tanh (no statistic of the row), whose mixers are linear attention with a constant decay per head ("lightning") or
// softmax attention through a latent under a sliding window ("latent_attention"), and of which a stretch of layers
// may run several times in a row with the same weights.
//
//     e = DyT(embed[token]; embed.norm)                          DyT(a; n) = tanh(alpha_n a) * w_n + b_n
//     a layer:  h = DyT(x; norm1);  x <- x + mixer(h) + ff(h)
//     before pass t of the stretch [loop.start, loop.stop):  x <- W_in [x ; e] + step[t]
//     logits = embed DyT(x; final.norm)                          the head is the embedding table
//
// config.json keys, all read here and nowhere else:
//   architecture ("Zerusun"), vocab, width, norm.eps, layers[i].type ("lightning" | "latent_attention"),
//   layers[i].mixer, layers[i].mlp (null: the layer has no feed-forward), loop {start, stop, times} (optional);
//   a lightning mixer: heads, dim, vdim, decay [heads];
//   a latent_attention mixer: heads, dim, rot_dim, vdim, q_rank, kv_rank, scale, mask {size} (optional: every earlier
//     position is seen), rot {base, dims, scaling {factor, original, fast, slow} (optional)};
//   mlp.kind "dense": ff;  mlp.kind "moe": expert {ff}, router {experts, top, scale (optional), groups {count, keep}
//     (optional)}, shared {ff} (optional);
//   max_position (optional): the longest sequence the rotary table is made for.
// Tensor names: embed, embed.norm{, .b, .alpha}, final.norm{, .b, .alpha}, loop.in, loop.step, and per layer i:
// l<i>.norm1{, .b, .alpha}; l<i>.mix.{q, k, v, g, o, norm} or l<i>.mix.{dq, dq.norm, uq, dkv, dkv.norm, uk, uv, g, o};
// l<i>.mlp.{gate, up, down} or l<i>.mlp.{router, e<j>.gate, e<j>.up, e<j>.down, shared.gate, shared.up, shared.down, shared.sg}.
//
// What the design fixes and the code therefore states: the dense unit's gate is the tanh form of gelu and the experts'
// (the shared one's too) silu; router scores are a softmax over all experts, a group counts as its best score, the
// chosen scores are divided by their sum and multiplied by router.scale; the shared expert's sum is multiplied by a
// sigmoid per token; the latent mixer's heads are gated by a sigmoid each; rotary pairs are (i, i + dims/2).
#include "config.h"

namespace qe {

namespace {
constexpr long long kDefaultMaxPosition = 65536;
const char* const kDenseActivation = "gelu_tanh";

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
}  // namespace

class ZerusunConfig : public ModelConfig {
public:
    Json source;                        // config.json as read (checked)
    long long vocab = 0, width = 0, max_position = kDefaultMaxPosition;
    long long loop_start = 0, loop_stop = 0, loop_times = 0;        // times 0: no stretch is repeated
    double eps = 0.0;

    static std::unique_ptr<ModelConfig> read(const Json& d) {
        std::unique_ptr<ZerusunConfig> c(new ZerusunConfig());
        c->architecture = "Zerusun";
        c->source = d;
        c->vocab = take_int(d, "vocab");
        c->width = take_int(d, "width");
        c->eps = take_float(object_at(d, "norm", ""), "eps");
        c->max_position = take_int(d, "max_position", kDefaultMaxPosition, 1);
        const Json* layers = d.find("layers");
        if (!layers || !layers->is_array() || layers->size() == 0) throw ConfigError("config.json: 'layers' must be a non-empty list");
        for (size_t i = 0; i < layers->size(); i++) {
            const Json& l = (*layers)[i];
            const std::string where = "layers[" + std::to_string(i) + "].";
            if (!l.is_object()) throw ConfigError("config.json: " + where + " must be an object");
            const std::string type = l.get_string("type", "");
            const Json& m = object_at(l, "mixer", where);
            if (type == "lightning") {
                const long long heads = take_int(m, "heads");
                take_int(m, "dim"); take_int(m, "vdim");
                const Json* decay = m.find("decay");
                if (!decay || !decay->is_array() || (long long)decay->size() != heads)
                    throw ConfigError("config.json: " + where + "mixer.decay must list one number per head");
                for (const Json& v : decay->items())
                    if (!v.is_number() || !(v.as_double() > 0.0) || v.as_double() > 1.0)
                        throw ConfigError("config.json: " + where + "mixer.decay: every decay lies in (0, 1]");
            } else if (type == "latent_attention") {
                take_int(m, "heads"); take_int(m, "dim"); take_int(m, "vdim"); take_int(m, "q_rank"); take_int(m, "kv_rank");
                const long long rot_dim = take_int(m, "rot_dim", 0);
                take_float(m, "scale");
                if (has_value(m, "mask")) take_int(object_at(m, "mask", where + "mixer."), "size");
                if (rot_dim > 0) {
                    const Json& rot = object_at(m, "rot", where + "mixer.");
                    const long long dims = take_int(rot, "dims", 2);
                    if (dims % 2 || dims > rot_dim) throw ConfigError("config.json: " + where + "mixer.rot.dims must be even and at most rot_dim");
                    if (!(take_float(rot, "base") > 1.0)) throw ConfigError("config.json: " + where + "mixer.rot.base must be above 1");
                    if (has_value(rot, "scaling")) {
                        const Json& sc = object_at(rot, "scaling", where + "mixer.rot.");
                        for (const char* key : {"factor", "original", "fast", "slow"})
                            if (!(take_float(sc, key) > 0)) throw ConfigError("config.json: " + where + "mixer.rot.scaling." + key + " must be positive");
                    }
                }
            } else {
                throw ConfigError("config.json: " + where + "type '" + type + "' is not known (lightning, latent_attention)");
            }
            if (has_value(l, "mlp")) {
                const Json& f = object_at(l, "mlp", where);
                const std::string kind = f.get_string("kind", "");
                if (kind == "dense") {
                    take_int(f, "ff");
                } else if (kind == "moe") {
                    take_int(object_at(f, "expert", where + "mlp."), "ff");
                    const Json& r = object_at(f, "router", where + "mlp.");
                    const long long experts = take_int(r, "experts"), top = take_int(r, "top");
                    take_float(r, "scale", 1.0);
                    long long count = 1, keep = 1;
                    if (has_value(r, "groups")) {
                        const Json& g = object_at(r, "groups", where + "mlp.router.");
                        count = take_int(g, "count");
                        keep = take_int(g, "keep");
                    }
                    if (top > experts || experts % count || keep > count || keep * (experts / count) < top)
                        throw ConfigError("config.json: " + where + "mlp.router: top " + std::to_string(top) + " of " + std::to_string(experts) +
                                          " experts in " + std::to_string(keep) + " of " + std::to_string(count) + " groups cannot be chosen");
                    if (has_value(f, "shared")) take_int(object_at(f, "shared", where + "mlp."), "ff");
                } else {
                    throw ConfigError("config.json: " + where + "mlp.kind '" + kind + "' is not known (dense, moe)");
                }
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
        d.set("architecture", "Zerusun");
        return d;
    }

    ModelSpec build_spec() const override {
        auto norm = [&](const std::string& name) {
            Json p = Json::object();
            p.set("size", width);
            p.set("names", names({{"weight", name}, {"bias", name + ".b"}, {"alpha", name + ".alpha"}}));
            return PartSpec("dyntanh", p);
        };
        auto gated_unit = [&](long long ff, const std::string& prefix, const char* activation) {
            Json g = Json::object();
            g.set("hidden_size", width);
            g.set("intermediate_size", ff);
            if (activation) {
                Json a = Json::object();
                a.set("kind", activation);
                g.set("activation", a);
            }
            g.set("names", names({{"gate_proj", prefix + "gate"}, {"up_proj", prefix + "up"}, {"down_proj", prefix + "down"}}));
            return PartSpec("swiglu", g);
        };
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
            layer.arrangement = "parallel";
            layer.parts.push_back({"norm", norm(p + "norm1")});
            if (l.at("type").as_string() == "lightning") {
                Json a = Json::object();
                a.set("hidden_size", width);
                a.set("num_heads", m.at("heads"));
                a.set("head_dim", m.at("dim"));
                a.set("value_dim", m.at("vdim"));
                a.set("decay", m.at("decay"));
                a.set("norm_eps", eps);
                a.set("names", names({{"q_proj", mp + "q"}, {"k_proj", mp + "k"}, {"v_proj", mp + "v"}, {"g_proj", mp + "g"}, {"o_proj", mp + "o"},
                                      {"norm", mp + "norm"}}));
                layer.parts.push_back({"mixer", PartSpec("lightning_attention", a)});
            } else {
                const long long rot_dim = take_int(m, "rot_dim", 0);
                Json a = Json::object();
                a.set("hidden_size", width);
                a.set("num_heads", m.at("heads"));
                a.set("head_dim", m.at("dim"));
                a.set("rot_dim", rot_dim);
                a.set("value_dim", m.at("vdim"));
                a.set("q_rank", m.at("q_rank"));
                a.set("kv_rank", m.at("kv_rank"));
                a.set("norm_eps", eps);
                a.set("scale", m.at("scale"));
                a.set("window", has_value(m, "mask") ? m.at("mask").at("size") : Json(0));
                a.set("gate", true);
                if (rot_dim > 0) {
                    const Json& rot = m.at("rot");
                    Json pos = Json::object();
                    pos.set("theta", rot.at("base"));
                    pos.set("n_rot", rot.at("dims"));
                    pos.set("max_position", max_position);
                    pos.set("pairing", "half");
                    if (has_value(rot, "scaling")) {
                        Json sc = rot.at("scaling");
                        sc.set("kind", "yarn");
                        pos.set("scaling", sc);
                    }
                    a.set("position", PartSpec("rope_neox", pos).to_json());
                } else {
                    a.set("position", Json());
                }
                a.set("names", names({{"q_down", mp + "dq"}, {"q_norm", mp + "dq.norm"}, {"q_up", mp + "uq"}, {"kv_down", mp + "dkv"},
                                      {"kv_norm", mp + "dkv.norm"}, {"k_up", mp + "uk"}, {"v_up", mp + "uv"}, {"o_proj", mp + "o"},
                                      {"gate", mp + "g"}}));
                layer.parts.push_back({"mixer", PartSpec("latent_attention", a)});
            }
            if (has_value(l, "mlp")) {
                const Json& f = l.at("mlp");
                const std::string fp = p + "mlp.";
                if (f.at("kind").as_string() == "dense") {
                    layer.parts.push_back({"feed_forward", gated_unit(f.at("ff").as_int(), fp, kDenseActivation)});
                } else {
                    const Json& router = f.at("router");
                    const long long experts = router.at("experts").as_int();
                    Json g = Json::object();
                    g.set("hidden_size", width);
                    g.set("intermediate_size", f.at("expert").at("ff"));
                    g.set("experts", experts);
                    g.set("top", router.at("top"));
                    Json scoring = Json::object();
                    scoring.set("kind", "softmax");
                    scoring.set("groups", has_value(router, "groups") ? router.at("groups").at("count") : Json(1));
                    scoring.set("keep", has_value(router, "groups") ? router.at("groups").at("keep") : Json(1));
                    scoring.set("scale", take_float(router, "scale", 1.0));
                    g.set("scoring", scoring);
                    Json n = names({{"router", fp + "router"}});
                    if (has_value(f, "shared")) {
                        n.set("shared_gate", fp + "shared.sg");
                        g.set("shared", gated_unit(f.at("shared").at("ff").as_int(), fp + "shared.", nullptr).to_json());
                    }
                    g.set("names", n);
                    Json list = Json::array();
                    for (long long e = 0; e < experts; e++) {
                        const std::string ep = fp + "e" + std::to_string(e) + ".";
                        list.push(names({{"gate_proj", ep + "gate"}, {"up_proj", ep + "up"}, {"down_proj", ep + "down"}}));
                    }
                    g.set("expert_names", list);
                    layer.parts.push_back({"feed_forward", PartSpec("routed_glu", g)});
                }
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
        e.set("norm", norm("embed.norm").to_json());
        e.set("names", names({{"weight", "embed"}}));
        spec.embedding = PartSpec("embedding", e);
        Json h = Json::object();
        h.set("hidden_size", width);
        h.set("vocab_size", vocab);
        h.set("tied_to", "embed");
        spec.head = PartSpec("lm_head", h);
        spec.final_norm = norm("final.norm");
        spec.validate();
        return spec;
    }
};

void register_zerusun_architecture() { register_architecture("Zerusun", ZerusunConfig::read); }

}  // namespace qe
