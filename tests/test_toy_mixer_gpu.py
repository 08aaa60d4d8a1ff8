"""A mixer with state of its own, defined here, is registered, built into a
model of a toy architecture (also defined here), given random weights, and
stepped through the engine in portions and mixed batches, with no change to
the package's files."""
from dataclasses import dataclass

import numpy as np
import pytest
import torch

import traces
from tolerances import check_close

pytestmark = pytest.mark.gpu


def _register():
    from cellm_b200.config import LayerSpec, ModelPlan, OrderEntry, PartSpec, register_architecture
    from cellm_b200.parts import FixedState, Mixer, TensorSpec, register_mixer

    class DecaySum(Mixer):
        """s_t = decay * s_(t-1) + W_in x_t ;  y_t = W_out (s_t * x_t). The state s
        (one vector per request) lives in a slot of the cache manager."""

        @classmethod
        def weight_specs(cls, p):
            return {"w_in": TensorSpec((p["state"], p["hidden_size"]), "linear"),
                    "w_out": TensorSpec((p["hidden_size"], p["state"]), "linear")}

        @classmethod
        def cache_need(cls, p):
            return FixedState((p["state"],), torch.float32)

        def __init__(self, params, weights, dtype):
            self.decay, self.w_in, self.w_out, self.dtype = params["decay"], weights["w_in"].float(), weights["w_out"].float(), dtype
            self.pick = torch.nn.functional.pad(torch.eye(params["state"], device=self.w_in.device), (0, params["hidden_size"] - params["state"]))

        def forward(self, x, ctx, cache):
            u = x.float() @ self.w_in.T
            out = torch.empty_like(u)
            o = 0
            for b, n in enumerate(ctx.q_lens):                      # portions of different requests, one after the other
                slot = int(ctx.slot_ids[b])
                s = cache.state[slot].clone()
                for i in range(n):
                    s = self.decay * s + u[o + i]
                    out[o + i] = s
                cache.state[slot] = s
                o += n
            return ((out * (x.float() @ self.pick.T)) @ self.w_out.T).to(self.dtype)

    register_mixer("toy_decay_sum", DecaySum)

    @dataclass(frozen=True)
    class ToyConfig:
        vocab: int
        width: int
        state: int
        decay: float
        eps: float

        @classmethod
        def from_dict(cls, d):
            return cls(d["toy_vocab"], d["toy_width"], d["toy_state"], d["toy_decay"], d["toy_eps"])

        def to_dict(self):
            return {"architectures": ["ToyDecayForCausalLM"], "toy_vocab": self.vocab, "toy_width": self.width,
                    "toy_state": self.state, "toy_decay": self.decay, "toy_eps": self.eps}

    def build_plan(c):
        norm = lambda name: PartSpec("rms_norm", {"dim": c.width, "eps": c.eps}, {"weight": name})
        layers = []
        for l in range(3):
            p = f"toy.{l}."
            if l == 1:       # a layer of the package's own attention between two toy layers
                mixer = PartSpec("attention", {"hidden_size": c.width, "num_heads": 2, "num_kv_heads": 1, "head_dim": 16,
                                               "scale": 0.25, "window": 0, "qk_norm": None,
                                               "position": PartSpec("rope", {"head_dim": 16, "rotary_dim": 16, "theta": 1e4, "layout": "half"})},
                                 {k: p + k for k in ("q_proj", "k_proj", "v_proj", "out_proj")})
            else:
                mixer = PartSpec("toy_decay_sum", {"hidden_size": c.width, "state": c.state, "decay": c.decay},
                                 {"w_in": p + "w_in", "w_out": p + "w_out"})
            ffn = PartSpec("swiglu", {"hidden_size": c.width, "ff_dim": 2 * c.width}, {k: p + "ffn." + k for k in ("w1", "w2", "w3")})
            layers.append(LayerSpec("pre_norm", mixer, ffn, norm(p + "n1"), norm(p + "n2")))
        return ModelPlan(hidden_size=c.width, vocab_size=c.vocab, max_positions=512, embedding="toy.embed",
                         final_norm=norm("toy.final"), head="toy.head", layers=tuple(layers),
                         order=tuple(OrderEntry(i) for i in range(3)))

    register_architecture("ToyDecayForCausalLM", ToyConfig, build_plan)


def toy_reference(folder, ids):
    """The same toy model, plainly, for a whole sequence in float64."""
    import json, os
    import plain_lfm2 as plain
    from safetensors.torch import load_file
    d = json.load(open(os.path.join(folder, "config.json")))
    w = {k: v.double() for k, v in load_file(os.path.join(folder, "model.safetensors")).items()}
    eps, decay, S = d["toy_eps"], d["toy_decay"], d["toy_state"]
    x = w["toy.embed"][torch.as_tensor(ids)]
    for l in range(3):
        p = f"toy.{l}."
        xn = plain.rms_norm(x, w[p + "n1"], eps)
        if l == 1:
            hd = 16
            mix, _ = plain.attention_mixer(xn, w[p + "q_proj"], w[p + "k_proj"], w[p + "v_proj"], w[p + "out_proj"],
                                           torch.ones(hd, dtype=torch.float64), torch.ones(hd, dtype=torch.float64),
                                           n_heads=2, n_kv=1, hd=hd, eps=0.0, theta=1e4)
            # no head norm in the toy: undo the unit-weight norm the plain function applies
            q = (xn @ w[p + "q_proj"].T).reshape(-1, 2, hd)
            k = (xn @ w[p + "k_proj"].T).reshape(-1, 1, hd)
            v = (xn @ w[p + "v_proj"].T).reshape(-1, 1, hd)
            pos = torch.arange(len(ids))
            q, k = plain.rope_rotate_half(q, pos, 1e4), plain.rope_rotate_half(k, pos, 1e4)
            out = torch.zeros(len(ids), 2, hd, dtype=torch.float64)
            for h in range(2):
                s = (q[:, h] @ k[:, 0].T) * 0.25
                s = s.masked_fill(torch.triu(torch.ones(len(ids), len(ids), dtype=torch.bool), 1), float("-inf"))
                out[:, h] = torch.softmax(s, -1) @ v[:, 0]
            mix = out.reshape(len(ids), -1) @ w[p + "out_proj"].T
        else:
            u = xn @ w[p + "w_in"].T
            s, rows = torch.zeros(S, dtype=torch.float64), []
            for t in range(len(ids)):
                s = decay * s + u[t]
                rows.append(s * xn[t, :S])
            mix = torch.stack(rows) @ w[p + "w_out"].T
        x = x + mix
        x = x + plain.swiglu(plain.rms_norm(x, w[p + "n2"], eps), w[p + "ffn.w1"], w[p + "ffn.w3"], w[p + "ffn.w2"])
    return (plain.rms_norm(x, w["toy.final"], eps) @ w["toy.head"].T).numpy()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_mixer_with_its_own_state_steps_through_the_engine(tmp_path, dtype):
    _register()
    from cellm_b200.replay import Replayer
    from cellm_b200.weights import InitSpec, write_random_model
    cfg = {"architectures": ["ToyDecayForCausalLM"], "toy_vocab": 300, "toy_width": 48, "toy_state": 24, "toy_decay": 0.9, "toy_eps": 1e-5}
    folder = write_random_model(str(tmp_path / "toy"), cfg, seed=4, dtype="bfloat16",
                                init=InitSpec(linear_std=0.15, embedding_std=0.3))
    rng = np.random.default_rng(2)
    reqs = {f"r{i}": rng.integers(0, 300, n).tolist() for i, n in enumerate((40, 9, 70, 3))}
    ref = {r: toy_reference(folder, t) for r, t in reqs.items()}
    for make in (traces.whole, traces.tail_one_by_one, traces.portions, traces.mixed):
        steps = make(reqs)
        rp = Replayer(folder, dtype, traces.max_live_tokens(steps), 8, 4)
        assert len(rp.cache.states) == 1 and tuple(rp.cache.states[0].shape) == (2, 4, 24)     # two toy layers, four slots
        got = traces.collect(steps, [rp.step(s["entries"], s["end"]) for s in steps])
        for r, t in reqs.items():
            check_close(traces.as_matrix(got[r], len(t)), ref[r], dtype, f"{make.__name__} {r}")


def test_toy_model_generates_through_the_engine(tmp_path):
    _register()
    from cellm_b200 import Engine, SamplingParams
    from cellm_b200.weights import InitSpec, write_random_model
    cfg = {"architectures": ["ToyDecayForCausalLM"], "toy_vocab": 300, "toy_width": 48, "toy_state": 24, "toy_decay": 0.9, "toy_eps": 1e-5}
    folder = write_random_model(str(tmp_path / "toy"), cfg, seed=4, dtype="bfloat16", init=InitSpec(linear_std=0.15, embedding_std=0.3))
    eng = Engine(folder, dtype="float32", tokens_per_block=8, total_blocks=32, max_num_seqs=2, max_batch_tokens=16, prefill_chunk=8)
    prompts = [[5, 9, 200, 7, 7, 31, 150, 2, 99, 100, 11], [42]]
    outs = eng.generate(prompts, SamplingParams.greedy(10, stop_eos=False))
    for p, o in zip(prompts, outs):
        toks = list(p)
        for t in o:
            lg = toy_reference(folder, toks)[-1]
            top = np.sort(lg)[-2:]
            assert t == int(lg.argmax()) or top[1] - top[0] < 1e-3 * (1 + np.abs(lg).max())
            toks.append(t)
