"""Llama model description shared by the engine binding, the synthetic-weight generator and the
benchmark: ``Config`` (ug_llama::model::Config, ug-llama/src/model.rs:10-24), the safetensors weight
names in load order (model.rs:313-346) and their shapes.  Pure Python: importing this module does not
load the CUDA library.
"""
from dataclasses import dataclass


@dataclass
class Config:
    """ug_llama::model::Config (ug-llama/src/model.rs:10-24)."""
    hidden_size: int
    intermediate_size: int
    max_position_embeddings: int
    num_attention_heads: int
    num_key_value_heads: int
    num_hidden_layers: int
    vocab_size: int
    rms_norm_eps: float = 1e-5
    rope_theta: float = 10000.0
    rope_interleaved: bool = False
    tie_word_embeddings: bool = True

    def head_dim(self):
        return self.hidden_size // self.num_attention_heads

    @staticmethod
    def from_json(path):
        """A Hugging Face ``config.json`` (what ug-llama deserialises into Config, main.rs:105-122)."""
        import json
        with open(path) as f:
            d = json.load(f)
        keys = ("hidden_size", "intermediate_size", "max_position_embeddings", "num_attention_heads",
                "num_key_value_heads", "num_hidden_layers", "vocab_size", "rms_norm_eps", "rope_theta",
                "rope_interleaved", "tie_word_embeddings")
        return Config(**{k: d[k] for k in keys if k in d})

    @staticmethod
    def llama_1b():
        """The Llama-1.1B shape of the benchmark configuration."""
        return Config(hidden_size=2048, intermediate_size=5632, max_position_embeddings=4096,
                      num_attention_heads=32, num_key_value_heads=4, num_hidden_layers=22,
                      vocab_size=32000)


def weight_names(cfg):
    """Tensor names in the order Model::new loads them (model.rs:313-346)."""
    names = ["model.embed_tokens.weight", "model.norm.weight"]
    for i in range(cfg.num_hidden_layers):
        p = f"model.layers.{i}"
        names += [f"{p}.input_layernorm.weight", f"{p}.post_attention_layernorm.weight",
                  f"{p}.mlp.gate_proj.weight", f"{p}.mlp.up_proj.weight", f"{p}.mlp.down_proj.weight",
                  f"{p}.self_attn.q_proj.weight", f"{p}.self_attn.k_proj.weight",
                  f"{p}.self_attn.v_proj.weight", f"{p}.self_attn.o_proj.weight"]
    return names


def weight_shape(cfg, name):
    h, f, kv = cfg.hidden_size, cfg.intermediate_size, cfg.head_dim() * cfg.num_key_value_heads
    if name == "model.embed_tokens.weight":
        return (cfg.vocab_size, h)
    if name.endswith("norm.weight"):
        return (h,)
    tail = name.split(".")[-2]
    return {"q_proj": (h, h), "k_proj": (kv, h), "v_proj": (kv, h), "o_proj": (h, h),
            "gate_proj": (f, h), "up_proj": (f, h), "down_proj": (h, f)}[tail]
