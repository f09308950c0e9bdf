"""Model factory and parameter accounting (complexity_deep/models/utils.py:9-98)."""
from __future__ import annotations

from .config import ComplexityConfig
from .modeling import ComplexityModel

SIZE_PRESETS = {
    "tiny": ComplexityConfig.complexity_tiny,
    "20m": ComplexityConfig.complexity_20m,
    "small": ComplexityConfig.complexity_small,
    "150m": ComplexityConfig.complexity_150m,
    "350m": ComplexityConfig.complexity_350m,
    "1b": ComplexityConfig.complexity_1b,
}


def create_complexity_model(size: str = "150m", vocab_size: int = 100_000, **overrides
                            ) -> ComplexityModel:
    """Builds a model from a preset name; unknown override keys are ignored."""
    if size not in SIZE_PRESETS:
        raise ValueError(f"Unknown size '{size}'. Choose from {list(SIZE_PRESETS.keys())}")
    config = SIZE_PRESETS[size]()
    config.vocab_size = vocab_size
    for key, value in overrides.items():
        if hasattr(config, key):
            setattr(config, key, value)
    return ComplexityModel(config)


class PrefillGraph:
    """CUDA-graph replay of ``model(input_ids).logits`` for one fixed ``[batch, seq]`` shape.

    A prefill step launches ~250 kernels; with few tokens per GPU the host cannot always issue
    them as fast as the GPU retires them.  Capturing the forward once and replaying it removes
    that overhead.  The dispatch kernels are part of the captured graph, so every replay routes
    the ids it is given.  Not part of the reference's API.

        graph = PrefillGraph(model, batch=4, seq_len=2048)
        logits = graph(input_ids)        # the returned tensor is overwritten by the next call
    """

    def __init__(self, model: ComplexityModel, batch: int, seq_len: int, warmup: int = 2):
        import torch
        from ..core.token_routed_mlp import ROUTING_CACHE
        self.model = model
        device = next(model.parameters()).device
        if device.type != "cuda":
            raise RuntimeError("PrefillGraph needs the model on a CUDA device")
        self.static_ids = torch.zeros(batch, seq_len, dtype=torch.int64, device=device)
        stream = torch.cuda.Stream(device=device)
        stream.wait_stream(torch.cuda.current_stream(device))
        with torch.no_grad(), torch.cuda.stream(stream):
            for _ in range(warmup):       # builds the packed weights, sets kernel attributes
                model(self.static_ids)
        torch.cuda.current_stream(device).wait_stream(stream)
        torch.cuda.synchronize(device)
        # a fresh version of the static buffer: the capture must contain the dispatch kernels,
        # not a cached result of the warm-up
        self.static_ids.add_(0)
        ROUTING_CACHE.clear()
        self.graph = torch.cuda.CUDAGraph()
        with torch.no_grad(), torch.cuda.graph(self.graph):
            self.static_logits = model(self.static_ids).logits
        ROUTING_CACHE.clear()             # its entries point into the graph's private pool

    def __call__(self, input_ids):
        self.static_ids.copy_(input_ids, non_blocking=True)
        self.graph.replay()
        return self.static_logits


def count_parameters(config: ComplexityConfig) -> dict:
    """Analytic parameter counts per component (shared expert as wide as one routed expert)."""
    H, I, V, L = (config.hidden_size, config.intermediate_size, config.vocab_size,
                  config.num_hidden_layers)
    hq, hkv = config.num_attention_heads, config.num_key_value_heads
    D = H // hq
    q_dim, kv_dim = hq * D, hkv * D

    qkv = q_dim * H + 2 * kv_dim * H
    attention = qkv + H * H                      # + o_proj
    if config.use_mu_guidance:
        attention += qkv                         # mu_to_q / k / v
    if config.use_qk_norm:
        attention += 2 * D

    if config.use_token_routed_mlp:
        E = config.num_experts
        per_expert = 3 * H * (I // E)
        mlp = E * per_expert + (per_expert if config.shared_expert else 0)
    else:
        mlp = 3 * H * I

    mu = H + H * H if config.use_mu_guidance else 0
    per_layer = attention + mlp + 2 * H + mu
    embedding = V * H
    total = embedding + L * per_layer + H
    return {
        "total": total,
        "embedding": embedding,
        "per_layer": per_layer,
        "attention_per_layer": attention,
        "mlp_per_layer": mlp,
        "mu_per_layer": mu,
        "num_layers": L,
        "memory_bf16_gb": total * 2 / (1024 ** 3),
    }
