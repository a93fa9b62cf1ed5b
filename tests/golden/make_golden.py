"""Generates tests/golden/*.npz.  Run from the repository root:

    python tests/golden/make_golden.py

The reference holds no expected outputs for this path (its only fixture is the input file
examples/data/bert_bs1.npy), so the golden outputs come from an independent implementation
of the same public model definition: `transformers`' PyTorch BertModel, built offline from a
config and loaded with the seeded synthetic weights of mononn_b200.models.  The CPU
restatement in oracle/ is pinned against these files.
"""
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from mononn_b200.models import (ClipConfig, EncoderConfig, clip_tiny, make_clip_inputs, make_inputs,  # noqa: E402
                                make_t5_inputs, make_vit_inputs, make_weights)

HERE = os.path.dirname(os.path.abspath(__file__))


def hf_bert_forward(cfg: EncoderConfig, w: dict, inputs: dict) -> np.ndarray:
    from transformers import BertConfig, BertModel
    hc = BertConfig(vocab_size=cfg.vocab, hidden_size=cfg.hidden, num_hidden_layers=cfg.layers,
                    num_attention_heads=cfg.heads, intermediate_size=cfg.ffn, hidden_act="gelu",
                    max_position_embeddings=cfg.max_pos, type_vocab_size=cfg.types,
                    layer_norm_eps=cfg.eps, hidden_dropout_prob=0.0, attention_probs_dropout_prob=0.0)
    model = BertModel(hc, add_pooling_layer=False).eval()
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a))
    sd = {
        "embeddings.word_embeddings.weight": t(w["embeddings.word"]),
        "embeddings.position_embeddings.weight": t(w["embeddings.position"]),
        "embeddings.token_type_embeddings.weight": t(w["embeddings.token_type"]),
        "embeddings.LayerNorm.weight": t(w["embeddings.ln.gamma"]),
        "embeddings.LayerNorm.bias": t(w["embeddings.ln.beta"]),
    }
    for l in range(cfg.layers):
        p, q = f"layer{l}.", f"encoder.layer.{l}."
        for ours, theirs in (("attn.q", "attention.self.query"), ("attn.k", "attention.self.key"),
                             ("attn.v", "attention.self.value"), ("attn.o", "attention.output.dense"),
                             ("ffn.up", "intermediate.dense"), ("ffn.down", "output.dense")):
            sd[q + theirs + ".weight"] = t(w[p + ours + ".w"].T)  # torch Linear stores [out, in]
            sd[q + theirs + ".bias"] = t(w[p + ours + ".b"])
        sd[q + "attention.output.LayerNorm.weight"] = t(w[p + "attn.ln.gamma"])
        sd[q + "attention.output.LayerNorm.bias"] = t(w[p + "attn.ln.beta"])
        sd[q + "output.LayerNorm.weight"] = t(w[p + "ffn.ln.gamma"])
        sd[q + "output.LayerNorm.bias"] = t(w[p + "ffn.ln.beta"])
    missing, unexpected = model.load_state_dict(sd, strict=False)
    missing = [m for m in missing if "position_ids" not in m]
    assert not missing and not unexpected, (missing, unexpected)
    with torch.no_grad():
        out = model(input_ids=torch.from_numpy(inputs["input_ids"]).long(),
                    attention_mask=torch.from_numpy(inputs["attention_mask"]).long(),
                    token_type_ids=torch.from_numpy(inputs["token_type_ids"]).long()).last_hidden_state
    return out.reshape(cfg.batch * cfg.seq, cfg.hidden).numpy()


def hf_vit_forward(cfg: EncoderConfig, w: dict, inputs: dict) -> np.ndarray:
    from transformers import ViTConfig, ViTModel
    hc = ViTConfig(hidden_size=cfg.hidden, num_hidden_layers=cfg.layers, num_attention_heads=cfg.heads,
                   intermediate_size=cfg.ffn, hidden_act="gelu", image_size=cfg.image, patch_size=cfg.patch,
                   num_channels=cfg.channels, layer_norm_eps=cfg.eps, hidden_dropout_prob=0.0,
                   attention_probs_dropout_prob=0.0, qkv_bias=True)
    model = ViTModel(hc, add_pooling_layer=False).eval()
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a))
    sd = {
        "embeddings.cls_token": t(w["embeddings.cls"].reshape(1, 1, -1)),
        "embeddings.position_embeddings": t(w["embeddings.position"][None]),
        # ours is [out, ky, kx, in]; torch Conv2d wants [out, in, ky, kx]
        "embeddings.patch_embeddings.projection.weight": t(w["embeddings.patch.w"].transpose(0, 3, 1, 2)),
        "embeddings.patch_embeddings.projection.bias": t(w["embeddings.patch.b"]),
        "layernorm.weight": t(w["ln.gamma"]), "layernorm.bias": t(w["ln.beta"]),
    }
    for l in range(cfg.layers):
        p, q = f"layer{l}.", f"encoder.layer.{l}."
        for ours, theirs in (("attn.q", "attention.attention.query"), ("attn.k", "attention.attention.key"),
                             ("attn.v", "attention.attention.value"), ("attn.o", "attention.output.dense"),
                             ("ffn.up", "intermediate.dense"), ("ffn.down", "output.dense")):
            sd[q + theirs + ".weight"] = t(w[p + ours + ".w"].T)
            sd[q + theirs + ".bias"] = t(w[p + ours + ".b"])
        sd[q + "layernorm_before.weight"] = t(w[p + "ln1.gamma"])
        sd[q + "layernorm_before.bias"] = t(w[p + "ln1.beta"])
        sd[q + "layernorm_after.weight"] = t(w[p + "ln2.gamma"])
        sd[q + "layernorm_after.bias"] = t(w[p + "ln2.beta"])
    missing, unexpected = model.load_state_dict(sd, strict=False)
    assert not missing and not unexpected, (missing, unexpected)
    with torch.no_grad():
        out = model(pixel_values=torch.from_numpy(inputs["pixel_values"])).last_hidden_state
    return out.reshape(cfg.batch * cfg.seq, cfg.hidden).numpy()


def hf_opt_forward(cfg: EncoderConfig, w: dict, inputs: dict) -> np.ndarray:
    from transformers import OPTConfig, OPTForCausalLM
    hc = OPTConfig(vocab_size=cfg.vocab, hidden_size=cfg.hidden, ffn_dim=cfg.ffn, num_hidden_layers=cfg.layers,
                   num_attention_heads=cfg.heads, max_position_embeddings=cfg.max_pos,
                   word_embed_proj_dim=cfg.hidden, do_layer_norm_before=True, dropout=0.0,
                   activation_function="relu", layer_norm_elementwise_affine=True)
    model = OPTForCausalLM(hc).eval()
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a))
    sd = {"model.decoder.embed_tokens.weight": t(w["embeddings.word"]),
          "model.decoder.embed_positions.weight": t(w["embeddings.position"]),
          "model.decoder.final_layer_norm.weight": t(w["ln.gamma"]),
          "model.decoder.final_layer_norm.bias": t(w["ln.beta"]),
          "lm_head.weight": t(w["embeddings.word"])}
    for l in range(cfg.layers):
        p, q = f"layer{l}.", f"model.decoder.layers.{l}."
        for ours, theirs in (("attn.q", "self_attn.q_proj"), ("attn.k", "self_attn.k_proj"),
                             ("attn.v", "self_attn.v_proj"), ("attn.o", "self_attn.out_proj"),
                             ("ffn.up", "fc1"), ("ffn.down", "fc2")):
            sd[q + theirs + ".weight"] = t(w[p + ours + ".w"].T)
            sd[q + theirs + ".bias"] = t(w[p + ours + ".b"])
        sd[q + "self_attn_layer_norm.weight"] = t(w[p + "ln1.gamma"])
        sd[q + "self_attn_layer_norm.bias"] = t(w[p + "ln1.beta"])
        sd[q + "final_layer_norm.weight"] = t(w[p + "ln2.gamma"])
        sd[q + "final_layer_norm.bias"] = t(w[p + "ln2.beta"])
    missing, unexpected = model.load_state_dict(sd, strict=False)
    assert not missing and not unexpected, (missing, unexpected)
    with torch.no_grad():
        out = model(input_ids=torch.from_numpy(inputs["input_ids"]).long()).logits
    return out.reshape(cfg.batch * cfg.seq, cfg.vocab).numpy()


def hf_clip_forward(cfg, w: dict, inputs: dict) -> np.ndarray:
    from transformers import CLIPConfig, CLIPModel
    v, t = cfg.vision, cfg.text
    tc = dict(vocab_size=t.vocab, hidden_size=t.hidden, intermediate_size=t.ffn, num_hidden_layers=t.layers,
              num_attention_heads=t.heads, max_position_embeddings=t.max_pos, hidden_act="quick_gelu",
              layer_norm_eps=t.eps, eos_token_id=2, attention_dropout=0.0)
    vc = dict(hidden_size=v.hidden, intermediate_size=v.ffn, num_hidden_layers=v.layers,
              num_attention_heads=v.heads, image_size=v.image, patch_size=v.patch, hidden_act="quick_gelu",
              layer_norm_eps=v.eps, attention_dropout=0.0)
    model = CLIPModel(CLIPConfig(text_config=tc, vision_config=vc, projection_dim=cfg.proj)).eval()
    tt = lambda a: torch.from_numpy(np.ascontiguousarray(a))
    sd = {"logit_scale": torch.tensor(float(np.log(cfg.logit_scale))),
          "text_model.embeddings.token_embedding.weight": tt(w["text.embeddings.word"]),
          "text_model.embeddings.position_embedding.weight": tt(w["text.embeddings.position"]),
          "text_model.final_layer_norm.weight": tt(w["text.ln.gamma"]),
          "text_model.final_layer_norm.bias": tt(w["text.ln.beta"]),
          "text_projection.weight": tt(w["text.proj.w"].T),
          "vision_model.embeddings.class_embedding": tt(w["vision.embeddings.cls"].reshape(-1)),
          "vision_model.embeddings.patch_embedding.weight": tt(w["vision.embeddings.patch.w"].transpose(0, 3, 1, 2)),
          "vision_model.embeddings.position_embedding.weight": tt(w["vision.embeddings.position"]),
          "vision_model.pre_layrnorm.weight": tt(w["vision.pre_ln.gamma"]),
          "vision_model.pre_layrnorm.bias": tt(w["vision.pre_ln.beta"]),
          "vision_model.post_layernorm.weight": tt(w["vision.ln.gamma"]),
          "vision_model.post_layernorm.bias": tt(w["vision.ln.beta"]),
          "visual_projection.weight": tt(w["vision.proj.w"].T)}
    for tower, c, pre in (("vision.", v, "vision_model."), ("text.", t, "text_model.")):
        for l in range(c.layers):
            p, q = f"{tower}layer{l}.", f"{pre}encoder.layers.{l}."
            for ours, theirs in (("attn.q", "self_attn.q_proj"), ("attn.k", "self_attn.k_proj"),
                                 ("attn.v", "self_attn.v_proj"), ("attn.o", "self_attn.out_proj"),
                                 ("ffn.up", "mlp.fc1"), ("ffn.down", "mlp.fc2")):
                sd[q + theirs + ".weight"] = tt(w[p + ours + ".w"].T)
                sd[q + theirs + ".bias"] = tt(w[p + ours + ".b"])
            for ours, theirs in (("ln1", "layer_norm1"), ("ln2", "layer_norm2")):
                sd[q + theirs + ".weight"] = tt(w[p + ours + ".gamma"])
                sd[q + theirs + ".bias"] = tt(w[p + ours + ".beta"])
    missing, unexpected = model.load_state_dict(sd, strict=False)
    missing = [m for m in missing if "position_ids" not in m]
    assert not missing and not unexpected, (missing, unexpected)
    with torch.no_grad():
        out = model(input_ids=torch.from_numpy(inputs["input_ids"]).long(),
                    pixel_values=torch.from_numpy(inputs["pixel_values"]))
    return out.logits_per_image.numpy()


def hf_t5_forward(cfg: EncoderConfig, w: dict, inputs: dict) -> np.ndarray:
    from transformers import T5Config, T5Model
    hc = T5Config(vocab_size=cfg.vocab, d_model=cfg.hidden, d_kv=cfg.hidden // cfg.heads, d_ff=cfg.ffn,
                  num_layers=cfg.layers, num_decoder_layers=cfg.layers, num_heads=cfg.heads,
                  relative_attention_num_buckets=32, relative_attention_max_distance=128, dropout_rate=0.0,
                  layer_norm_epsilon=cfg.eps, feed_forward_proj="relu", tie_word_embeddings=True)
    model = T5Model(hc).eval()
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a))
    sd = {"shared.weight": t(w["shared"]), "encoder.embed_tokens.weight": t(w["shared"]),
          "decoder.embed_tokens.weight": t(w["shared"])}
    for stack in ("encoder", "decoder"):
        sd[f"{stack}.block.0.layer.0.SelfAttention.relative_attention_bias.weight"] = t(w[f"{stack}.rel_bias"])
        sd[f"{stack}.final_layer_norm.weight"] = t(w[f"{stack}.ln.gamma"])
        for l in range(cfg.layers):
            p, q = f"{stack}.layer{l}.", f"{stack}.block.{l}.layer."
            ff = 1 if stack == "encoder" else 2
            for n in ("q", "k", "v", "o"):
                sd[f"{q}0.SelfAttention.{n}.weight"] = t(w[p + f"attn.{n}.w"].T)
                if stack == "decoder":
                    sd[f"{q}1.EncDecAttention.{n}.weight"] = t(w[p + f"xattn.{n}.w"].T)
            sd[f"{q}0.layer_norm.weight"] = t(w[p + "ln1.gamma"])
            if stack == "decoder":
                sd[f"{q}1.layer_norm.weight"] = t(w[p + "lnx.gamma"])
            sd[f"{q}{ff}.layer_norm.weight"] = t(w[p + "ln2.gamma"])
            sd[f"{q}{ff}.DenseReluDense.wi.weight"] = t(w[p + "ffn.up.w"].T)
            sd[f"{q}{ff}.DenseReluDense.wo.weight"] = t(w[p + "ffn.down.w"].T)
    missing, unexpected = model.load_state_dict(sd, strict=False)
    assert not missing and not unexpected, (missing, unexpected)
    with torch.no_grad():
        out = model(input_ids=torch.from_numpy(inputs["input_ids"]).long(),
                    decoder_input_ids=torch.from_numpy(inputs["decoder_input_ids"]).long()).last_hidden_state
    return out.reshape(cfg.batch * cfg.seq, cfg.hidden).numpy()


CASES = {
    # name: (config, weight seed, stress, pad_fraction)
    "bert_tiny_b1_s16": (EncoderConfig(layers=2, hidden=64, heads=1, ffn=256, vocab=100, max_pos=64,
                                       batch=1, seq=16), 11, True, 0.0),
    "bert_small_b2_s24_pad": (EncoderConfig(layers=2, hidden=128, heads=2, ffn=512, vocab=300, max_pos=64,
                                            batch=2, seq=24), 12, True, 0.25),
    "vit_tiny_b2_img48": (EncoderConfig(model="vit", layers=2, hidden=128, heads=2, ffn=256, batch=2, seq=10,
                                        image=48, patch=16, channels=3, max_pos=10, vocab=0, types=0),
                          13, True, 0.0),
    "opt_tiny_b2_s24": (EncoderConfig(model="opt", layers=2, hidden=128, heads=2, ffn=256, vocab=160, max_pos=64,
                                      types=0, batch=2, seq=24, eps=1e-5, act="relu"), 14, True, 0.0),
    "clip_tiny_i3_t5": (clip_tiny(images=3, texts=5, layers=2), 15, True, 0.0),
    "t5_tiny_b2_s32": (EncoderConfig(model="t5", layers=2, hidden=128, heads=2, ffn=256, vocab=96, max_pos=0,
                                     types=0, batch=2, seq=32, eps=1e-6, act="relu"), 16, True, 0.0),
}


def main():
    for name, (cfg, seed, stress, pad) in CASES.items():
        w = make_weights(cfg, seed, stress=stress)
        if cfg.model == "vit":
            inp = make_vit_inputs(cfg, seed)
            out = hf_vit_forward(cfg, w, inp)
        elif isinstance(cfg, ClipConfig):
            inp = make_clip_inputs(cfg, seed)
            out = hf_clip_forward(cfg, w, inp)  # logits_per_image; stored under the common key
        elif cfg.model == "t5":
            inp = make_t5_inputs(cfg, seed)
            out = hf_t5_forward(cfg, w, inp)  # the decoder's last hidden state
        elif cfg.model == "opt":
            inp = make_inputs(cfg, seed)
            out = hf_opt_forward(cfg, w, inp)  # logits; stored under the common key
        else:
            inp = make_inputs(cfg, seed, pad_fraction=pad)
            out = hf_bert_forward(cfg, w, inp)
        # keep the file small: the inputs are regenerated from the seed, only the output is stored
        np.savez_compressed(os.path.join(HERE, name + ".npz"), last_hidden_state=out.astype(np.float32),
                            seed=np.int64(seed), stress=np.bool_(stress), pad=np.float64(pad))
        print(name, out.shape, float(np.abs(out).mean()))


if __name__ == "__main__":
    main()
