"""Model zoo of the race driver and the benchmarks."""
from .llama import LLAMA_1P3B, LLAMA_TINY, Llama, LlamaConfig
from .mamba import MambaModel, SelectiveSSMLayer
from .transformer import DecoderBlock, PreLNTransformer, Transformer
from .vit import ViT

MODEL_SCALES = {
    "small": {"dim_model": 128, "num_heads": 4, "num_layers": 2},
    "medium": {"dim_model": 256, "num_heads": 8, "num_layers": 4},
    "large": {"dim_model": 512, "num_heads": 8, "num_layers": 6},
}


def build_model(cfg: dict):
    """Model for a race configuration dict (keys as in the reference DEFAULT_CONFIG, grokking_race_v2.py:219-228)."""
    mt = cfg.get("model_type", "decoder")
    nl, d, h = cfg.get("num_layers", 2), cfg.get("dim_model", 128), cfg.get("num_heads", 4)
    if mt == "decoder":
        return Transformer(nl, d, h, cfg.get("num_tokens", 99), cfg.get("seq_len_model", 4))
    if mt == "decoder_preln":
        return PreLNTransformer(nl, d, h, cfg.get("num_tokens", 99), cfg.get("seq_len_model", 4))
    if mt == "vit":
        return ViT(nl, d, h, cfg.get("p", 97), cfg.get("patch_dim", 49), cfg.get("num_patches", 16))
    if mt == "mamba":
        return MambaModel(nl, d, cfg.get("num_tokens", 99), 2 * cfg.get("chain_length", 3) + 2)
    raise ValueError(f"Unknown model_type: {mt}")
