"""The Linonex decoder: its name in config.json and the names of its tensors.

Layer i's tensors start with "l<i>."; a mixer's are "l<i>.mix.*" (the two sides of a parallel mixer under
"l<i>.mix.left.*" and "l<i>.mix.right.*"), a feed-forward's "l<i>.mlp.*" (expert e's "l<i>.mlp.e<e>.*"), the two norms
"l<i>.norm1" and "l<i>.norm2". The frame's are "embed", "pos", "final.norm" and "head".
"""
from ..config.linonex import LinonexConfig
from ..config.registry import register_architecture
from .layout import ModelLayout
from .model import expected_tensors

_MEMORY = {"wq": "q", "wk": "k", "wv": "v", "wg": "g", "wi": "i", "bi": "i.b", "wf": "f", "bf": "f.b", "out_norm": "norm",
           "wo": "o"}
_LEFT = {"wq": "q", "wk": "k", "wv": "v", "conv_q": "q.conv", "conv_k": "k.conv", "conv_v": "v.conv", "wo": "o"}
_RIGHT = {"wq": "q", "wk": "k", "wv": "v", "conv_q": "q.conv", "conv_k": "k.conv", "conv_v": "v.conv", "wb": "b", "wa": "a",
          "decay_log": "A_log", "decay_bias": "dt_bias", "wg": "g", "out_norm": "norm", "wo": "o"}


class LinonexArchitecture:
    name = "Linonex"

    def parse_config(self, raw):
        return LinonexConfig.from_dict(raw)

    def layout(self, spec):
        layers = []
        for l, block in enumerate(spec.layers):
            p = f"l{l}."
            names = {("mixer_norm", "weight"): p + "norm1"}
            if block.mixer.kind == "matrix_memory":
                for slot, short in _MEMORY.items():
                    names[("mixer", slot)] = p + "mix." + short
            else:
                for side, table in (("left", _LEFT), ("right", _RIGHT)):
                    for slot, short in table.items():
                        names[("mixer", f"{side}.{slot}")] = f"{p}mix.{side}.{short}"
                    names[("mixer", f"{side}_out")] = f"{p}mix.{side}.out"
            ffn = block.ffn
            if ffn is not None:
                names[("ffn_norm", "weight")] = p + "norm2"
                if ffn.kind == "routed_mlp":
                    names[("ffn", "router")] = p + "mlp.router"
                    names[("ffn", "correction")] = p + "mlp.correction"
                    for e in range(ffn.experts):
                        for slot in ("gate", "up", "down"):
                            names[("ffn", f"{slot}{e}")] = f"{p}mlp.e{e}.{slot}"
                else:
                    for slot in ("gate", "up", "down"):
                        names[("ffn", slot)] = p + "mlp." + slot
            layers.append(names)
        return ModelLayout(embed="embed", final_norm="final.norm", head="head", layers=layers, frame={"positions": "pos"})

    def random_moments(self, name, shape, std, norm_std):
        """(mean, amplitude) of a random tensor of this design where the general rule (matrices around zero, vectors
        around one) does not fit; None: the general rule."""
        last = name.rsplit(".", 1)[-1]
        if last in ("A_log", "dt_bias", "correction") or name.endswith((".i.b", ".f.b")):
            return (1.0 if name.endswith(".f.b") else 0.0), 0.5
        if last == "conv":
            return 0.0, 0.5
        return None

    def info(self, spec):
        kinds = "".join("m" if b.mixer.kind == "matrix_memory" else "p" for b in spec.layers)
        ffs = "".join("-" if b.ffn is None else "e" if b.ffn.kind == "routed_mlp" else "d" for b in spec.layers)
        return (f"linonex dim={spec.hidden} layers={len(spec.layers)} ({kinds}; feed-forwards {ffs}; "
                f"{len(spec.schedule)} layer runs) vocab={spec.vocab}")

    def tensor_names(self, spec, available=None):
        return expected_tensors(spec, self.layout(spec), available)


register_architecture(LinonexArchitecture())
