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


class DecodeGraph:
    """CUDA-graph replay of one decode step (one new token per sequence) on a StaticKVCache.

    A decode step of the 1B model is ~270 launches of a few microseconds each, so the step
    time is set by how fast the host can issue them.  The cache position is a device scalar
    (see ``StaticKVCache``), so one captured step serves every length; a replay costs one
    launch.  Steps attend to the whole cache (the reference's result for an all-zero additive
    mask).  Not part of the reference's API.

        dec = DecodeGraph(model, batch=32, capacity=prompt_len + max_new_tokens)
        logits = dec.prefill(prompt_ids)     # ordinary forward; its cache is copied in
        logits = dec.step(next_ids)          # [batch, 1, vocab], overwritten by the next step
    """

    def __init__(self, model: ComplexityModel, batch: int, capacity: int, warmup: int = 2):
        import torch
        from ..core.attention import StaticKVCache
        from ..core.token_routed_mlp import ROUTING_CACHE
        self.model = model
        cfg = model.config
        device = next(model.parameters()).device
        if device.type != "cuda":
            raise RuntimeError("DecodeGraph needs the model on a CUDA device")
        self.cache = StaticKVCache(cfg.num_hidden_layers, batch, cfg.num_key_value_heads,
                                   cfg.hidden_size // cfg.num_attention_heads, capacity, device,
                                   dtype=next(model.parameters()).dtype)
        self.static_ids = torch.zeros(batch, 1, dtype=torch.int64, device=device)
        stream = torch.cuda.Stream(device=device)
        stream.wait_stream(torch.cuda.current_stream(device))
        with torch.no_grad(), torch.cuda.stream(stream):
            for _ in range(warmup):       # builds the packed weights, sets kernel attributes
                self._eager_step()
        torch.cuda.current_stream(device).wait_stream(stream)
        torch.cuda.synchronize(device)
        self.static_ids.add_(0)           # fresh version: the capture must contain the dispatch
        ROUTING_CACHE.clear()
        self.graph = torch.cuda.CUDAGraph()
        with torch.no_grad(), torch.cuda.graph(self.graph):
            self.static_logits = self._eager_step()
        ROUTING_CACHE.clear()             # its entries point into the graph's private pool
        self.cache.set_length(0)          # the warm-up and capture steps wrote scratch rows

    def _eager_step(self):
        logits = self.model(self.static_ids, past_key_values=self.cache.layers,
                            use_cache=True).logits
        self.cache.state.add_(1)
        return logits

    def prefill(self, input_ids, attention_mask=None):
        """Runs the prompt through the model and moves its KV cache into the static buffers."""
        import torch
        with torch.no_grad():
            out = self.model(input_ids, attention_mask=attention_mask, use_cache=True)
        self.cache.load(out.past_key_values)
        return out.logits

    def step(self, input_ids):
        if self.cache.length >= self.cache.capacity:
            raise RuntimeError(f"KV cache full ({self.cache.capacity} tokens)")
        self.static_ids.copy_(input_ids.view(self.static_ids.shape), non_blocking=True)
        self.graph.replay()
        self.cache.length += 1
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
