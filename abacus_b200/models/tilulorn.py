"""The Tilulorn decoder: its name in config.json and the names of its tensors.

Layer i's tensors start with "l<i>."; a mixer's are "l<i>.mix.*", a feed-forward's "l<i>.mlp.*" (expert e's
"l<i>.mlp.e<e>.*", the table of experts by token id "l<i>.mlp.table"), the two norms "l<i>.norm1" and "l<i>.norm2".
The frame's are "embed", "final.norm", "head", and, where a run of layers is gone through in passes, "loop.in" and
"loop.step".
"""
from ..config.registry import register_architecture
from ..config.tilulorn import TilulornConfig
from .layout import ModelLayout
from .model import expected_tensors

_LATENT = {"wdq": "dq", "q_norm": "dq.norm", "wq": "uq", "wdown": "dkv", "down_norm": "dkv.norm", "wuk": "uk", "wuv": "uv",
           "wg": "g", "wo": "o"}
_WINDOWED = {"wq": "q", "wk": "k", "q_norm": "q.norm", "k_norm": "k.norm", "sink": "sink", "wg": "g", "wo": "o"}
_WKV = {"mu_r": "mu.r", "mu_k": "mu.k", "mu_v": "mu.v", "mu_g": "mu.g", "mu_w": "mu.w", "wr": "r", "wk": "k", "wv": "v",
        "wg": "g", "w1": "w1", "w2": "w2", "w0": "w0", "bonus": "u", "out_norm": "norm", "wo": "o"}
_BY_KIND = {"latent_attention": _LATENT, "attention": _WINDOWED, "wkv": _WKV}


class TilulornArchitecture:
    name = "Tilulorn"

    def parse_config(self, raw):
        return TilulornConfig.from_dict(raw)

    def complete_config(self, config, shapes):
        """Sizes that config.json leaves to the tensors, read from their shapes ({name: shape})."""
        return config.with_ranks(shapes)

    def layout(self, spec):
        layers = []
        for l, block in enumerate(spec.layers):
            p = f"l{l}."
            names = {("mixer_norm", "weight"): p + "norm1"}
            for slot, short in _BY_KIND[block.mixer.kind].items():
                names[("mixer", slot)] = p + "mix." + short
            ffn = block.ffn
            if ffn is not None:
                names[("ffn_norm", "weight")] = p + "norm2"
                names[("ffn", "table")] = p + "mlp.table"
                for e in range(ffn.experts):
                    for slot in ("gate", "up", "down"):
                        names[("ffn", f"{slot}{e}")] = f"{p}mlp.e{e}.{slot}"
            layers.append(names)
        return ModelLayout(embed="embed", final_norm="final.norm", head="head", layers=layers,
                           frame={"loop_in": "loop.in", "loop_step": "loop.step"})

    def random_moments(self, name, shape, std, norm_std):
        """(mean, amplitude) of a random tensor of this design where the general rule (matrices around zero, vectors
        around one) does not fit; None: the general rule."""
        last = name.rsplit(".", 1)[-1]
        if last in ("sink", "w0", "u", "step") or ".mu." in name:
            return (0.5 if ".mu." in name else 0.0), (0.25 if ".mu." in name else 0.5)
        return None

    def info(self, spec):
        kinds = "".join({"latent_attention": "l", "attention": "a", "wkv": "w"}[b.mixer.kind] for b in spec.layers)
        ffs = "".join("-" if b.ffn is None else "e" for b in spec.layers)
        return (f"tilulorn dim={spec.hidden} layers={len(spec.layers)} ({kinds}; feed-forwards {ffs}; "
                f"{len(spec.schedule)} layer runs) vocab={spec.vocab}")

    def tensor_names(self, spec, available=None):
        return expected_tensors(spec, self.layout(spec), available)


register_architecture(TilulornArchitecture())
