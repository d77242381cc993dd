"""Generate tests/golden/decoder_vectors.npz and decoder_ve_vectors.npz: logits of the reference's exported model
(inference/modeling_nanochat.py NanochatForCausalLM, bf16 weights, DynamicCache decode on CPU) on a tiny random-init
configuration, for the end-to-end decoder's parity tests.

    PYTHONPATH=<reference checkout> PYTHONDONTWRITEBYTECODE=1 python tests/golden/make_golden_decoder.py

Weights are regenerated in the tests from the same seeds (tests/helpers.py:tiny_decoder_weights and
tiny_decoder_weights_ve: the second adds a value-embedding layer and non-trivial stream-mix lambdas) and pinned here
by checksum. The run is: a 12-token prompt in one forward pass (prefill), then 6 greedy tokens one at a time with the
cache; logits of the last prompt position and of every decode step are stored."""

import hashlib
import sys
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parent.parent.parent
sys.path.insert(0, str(ROOT))

from inference import modeling_nanochat as ref  # noqa: E402  (the reference, from PYTHONPATH)

from tests import helpers  # noqa: E402

def run_reference(cfg: dict, weights: dict, name: str) -> None:
    L, C, H, Fd, V = cfg["n_layers"], cfg["hidden"], cfg["n_heads"], cfg["intermediate"], cfg["vocab"]
    ve_layers = [i for i, lw in enumerate(weights["layers"]) if lw.get("ve_table") is not None]
    config = ref.NanochatConfig(
        vocab_size=V, hidden_size=C, intermediate_size=Fd, num_hidden_layers=L, num_attention_heads=H,
        num_key_value_heads=H, head_dim=128, max_position_embeddings=256,
        rope_parameters={"rope_type": "default", "rope_theta": cfg["rope_theta"]}, sliding_window=257,
        layer_types=["full_attention"] * L, value_embedding_layers=ve_layers, final_logit_softcapping=15.0,
        rms_norm_eps=float(np.finfo(np.float32).eps), tie_word_embeddings=False, dtype="bfloat16",
        bos_token_id=0, eos_token_id=0)
    config._attn_implementation = "eager"
    model = ref.NanochatForCausalLM(config).to(torch.bfloat16).eval()
    resid = torch.tensor([lw.get("resid_lambda", 1.0) for lw in weights["layers"]])
    x0 = torch.tensor([lw.get("x0_lambda", 0.0) for lw in weights["layers"]])
    state = {"model.embed_tokens.weight": weights["embed"], "lm_head.weight": weights["lm_head"],
             "model.resid_lambdas": resid, "model.x0_lambdas": x0}
    for i, lw in enumerate(weights["layers"]):
        p = f"model.layers.{i}."
        q, k, v = lw["wqkv"].split(H * 128, dim=0)
        state.update({p + "self_attn.q_proj.weight": q, p + "self_attn.k_proj.weight": k,
                      p + "self_attn.v_proj.weight": v, p + "self_attn.o_proj.weight": lw["wo"],
                      p + "mlp.up_proj.weight": lw["wup"], p + "mlp.down_proj.weight": lw["wdown"],
                      p + "self_attn.q_norm_weight": lw["q_gain"], p + "self_attn.k_norm_weight": lw["k_gain"]})
        if i in ve_layers:
            state.update({f"model.value_embeds.{i}.weight": lw["ve_table"],
                          p + "self_attn.ve_gate.weight": lw["ve_gate"]})
    missing, unexpected = model.load_state_dict(state, strict=False)
    assert not unexpected and not missing, (missing, unexpected)
    for layer in model.model.layers:  # the reference keeps these in fp32
        for attr in ("q_norm_weight", "k_norm_weight"):
            setattr(layer.self_attn, attr, torch.nn.Parameter(getattr(layer.self_attn, attr).float()))
    for i in ve_layers:
        model.model.layers[i].self_attn.ve_gate.weight = torch.nn.Parameter(weights["layers"][i]["ve_gate"].float())
    model.model.resid_lambdas = torch.nn.Parameter(resid.float())
    model.model.x0_lambdas = torch.nn.Parameter(x0.float())

    gen = torch.Generator().manual_seed(11)
    prompt = torch.randint(0, V, (2, 12), generator=gen)
    with torch.no_grad():
        out = model(input_ids=prompt, use_cache=True)
        cache = out.past_key_values
        logits = [out.logits[:, -1]]
        tokens = []
        for _ in range(6):
            nxt = logits[-1].argmax(-1)
            tokens.append(nxt)
            out = model(input_ids=nxt[:, None], past_key_values=cache, use_cache=True)
            logits.append(out.logits[:, -1])

    digest = hashlib.sha256()
    for t in [weights["embed"], weights["lm_head"]] + [lw[k] for lw in weights["layers"] for k in sorted(lw)
                                                        if isinstance(lw[k], torch.Tensor)]:
        digest.update(t.contiguous().view(torch.uint8).numpy().tobytes())
    np.savez_compressed(Path(__file__).resolve().parent / name,
                        prompt=prompt.numpy(), tokens=torch.stack(tokens, 1).numpy(),
                        logits=torch.stack(logits, 1).float().numpy(),  # (2, 7, V): capped, c tanh(z / c)
                        softcap=np.float32(15.0), weights_sha256=np.frombuffer(digest.digest(), dtype=np.uint8))
    print(name, "tokens", torch.stack(tokens, 1).tolist(), "logit std", float(torch.stack(logits, 1).std()))


run_reference(*helpers.tiny_decoder_weights(), "decoder_vectors.npz")
# the reference's own model shape: a value embedding on the last layer and stream-mix lambdas away from (1, 0)
run_reference(*helpers.tiny_decoder_weights_ve(), "decoder_ve_vectors.npz")
