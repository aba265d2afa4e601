"""Shared test helpers: configurations named in BASELINE.json and seeded inputs."""
import numpy as np

# cfg 1: tiny synthetic hybrid MoE (GDN, GDN, GDN, full attention).
TINY = dict(n_layer=4, n_embd=256, n_head=4, n_head_kv=1, head_dim=64, n_vocab=1024, rope_theta=1e7, rms_eps=1e-6,
            n_rot=16, ssm_d_conv=4, ssm_d_inner=256, ssm_d_state=64, ssm_dt_rank=4, ssm_n_group=2,
            full_attention_interval=4, n_expert=16, n_expert_used=4, expert_ff=128, shared_ff=128)


def oracle_dims(d):
    from oracle import oracle_py as O
    return O.ModelDims(**d)


def prompt_ids(seed, n, n_vocab):
    """Uniform-random token ids from a seeded generator."""
    return np.random.default_rng(seed).integers(0, n_vocab, n).astype(np.uint32)


def noise(n, seed, scale=1.0):
    return (np.random.default_rng(seed).standard_normal(n) * scale).astype(np.float32)
