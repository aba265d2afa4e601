"""The synthetic model shapes BASELINE.json names (qwen35moe structure, src/model/qwen35.rs:193-249)."""

# cfg 1: tiny hybrid MoE, layers GDN, GDN, GDN, full attention. n_rot is hd/4, the 35B's 64/256 ratio.
TINY = dict(n_layer=4, n_embd=256, n_head=4, n_head_kv=1, head_dim=64, n_vocab=1024, rope_theta=1e7, rms_eps=1e-6,
            n_rot=16, ssm_d_conv=4, ssm_d_inner=256, ssm_d_state=64, ssm_dt_rank=4, ssm_n_group=2,
            full_attention_interval=4, n_expert=16, n_expert_used=4, expert_ff=128, shared_ff=128)

# A small shape whose every matrix has k a multiple of 256, so the pipelined multi-row kernels (which need that) run in tests.
MID = dict(n_layer=4, n_embd=512, n_head=4, n_head_kv=1, head_dim=64, n_vocab=1024, rope_theta=1e7, rms_eps=1e-6,
           n_rot=16, ssm_d_conv=4, ssm_d_inner=512, ssm_d_state=128, ssm_dt_rank=4, ssm_n_group=2,
           full_attention_interval=4, n_expert=64, n_expert_used=4, expert_ff=256, shared_ff=256)

# A small shape with the ~177B model's awkward ratios: widths that are 3 x a power of two (24 and 6 quantisation blocks per
# row), 10 picks, 3 query heads per kv head, 6 value heads on 3 key heads, head_dim 128, conv width 4.
ODD = dict(n_layer=4, n_embd=768, n_head=6, n_head_kv=2, head_dim=128, n_vocab=512, rope_theta=1e7, rms_eps=1e-6,
           n_rot=32, ssm_d_conv=4, ssm_d_inner=768, ssm_d_state=128, ssm_dt_rank=6, ssm_n_group=3,
           full_attention_interval=4, n_expert=48, n_expert_used=10, expert_ff=192, shared_ff=192)

# cfg 2-4: 35B-A3B shape. 40 layers (3 GDN : 1 attention), 256 experts top-8 + shared.
M35B = dict(n_layer=40, n_embd=2048, n_head=16, n_head_kv=2, head_dim=256, n_vocab=248320, rope_theta=1e7, rms_eps=1e-6,
            n_rot=64, ssm_d_conv=4, ssm_d_inner=4096, ssm_d_state=128, ssm_dt_rank=32, ssm_n_group=16,
            full_attention_interval=4, n_expert=256, n_expert_used=8, expert_ff=512, shared_ff=512)

# cfg 5: ~177B shape. 48 layers, 512 experts top-10 + shared.
L177B = dict(n_layer=48, n_embd=3072, n_head=32, n_head_kv=4, head_dim=256, n_vocab=248320, rope_theta=1e7, rms_eps=1e-6,
             n_rot=64, ssm_d_conv=4, ssm_d_inner=6144, ssm_d_state=128, ssm_dt_rank=48, ssm_n_group=16,
             full_attention_interval=4, n_expert=512, n_expert_used=10, expert_ff=768, shared_ff=768)

SEEDS = dict(tiny=0, mid=5, odd=6, m35b=3, l177b=4)


def with_layers(cfg, n_layer):
    """The same shape with fewer layers (bounded CPU samples and small-memory tests)."""
    c = dict(cfg); c["n_layer"] = n_layer
    return c
