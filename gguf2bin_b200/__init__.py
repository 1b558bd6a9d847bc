"""gguf2bin_b200: a small generation library for the Qwen3 dense architecture on one
B200 (sm_100a), put together from exchangeable parts.

    config/    typed configuration and the architecture registry
    weights/   safetensors reading, by-name binding, random-weights model writer
    parts/     norms, position encodings, mixers, feed-forwards, blocks
    cache/     sequence slots, token pages, per-slot state, storage per layer group
    engine/    model, step function, generation loop
    sampling/  greedy, temperature, top-k / top-p / repeat penalty
    csrc/      the CUDA kernels and their build
"""
__version__ = "0.1.0"
