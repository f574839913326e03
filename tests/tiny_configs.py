"""The tests' own tiny configurations of the architecture.  They differ in every size
and option: layers, width, head counts and groups (4/2, 3/1, 6/2), head sizes (16, 32, 48, 64, 128),
``num_heads * head_dim`` equal to the width or not, feed-forward width, vocabulary (a power
of two, a multiple of 128, odd), norm epsilon, rotary base, frequency scaling (none and two
llama3 blocks), tied and untied heads.  Weights are drawn wider than the usual 0.02 so that
attention is far from uniform: a misplaced key or position then changes the logits by far
more than any tolerance."""

A = dict(architectures=["LlamaForCausalLM"], vocab_size=256, hidden_size=64, intermediate_size=192,
         num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, head_dim=16,
         max_position_embeddings=512, rms_norm_eps=1e-5, rope_theta=10000.0, rope_scaling=None,
         tie_word_embeddings=True, eos_token_id=7)

B = dict(architectures=["LlamaForCausalLM"], vocab_size=384, hidden_size=96, intermediate_size=256,
         num_hidden_layers=3, num_attention_heads=3, num_key_value_heads=1, head_dim=32,
         max_position_embeddings=512, rms_norm_eps=1e-6, rope_theta=500000.0,
         rope_scaling=dict(rope_type="llama3", factor=8.0, low_freq_factor=1.0, high_freq_factor=4.0,
                           original_max_position_embeddings=16),
         tie_word_embeddings=False, eos_token_id=[5, 9])

C = dict(architectures=["LlamaForCausalLM"], vocab_size=301, hidden_size=72, intermediate_size=200,
         num_hidden_layers=4, num_attention_heads=6, num_key_value_heads=2, head_dim=48,
         max_position_embeddings=1024, rms_norm_eps=2e-5, rope_theta=1000000.0,
         rope_scaling=dict(rope_type="llama3", factor=4.0, low_freq_factor=1.0, high_freq_factor=2.0,
                           original_max_position_embeddings=32),
         tie_word_embeddings=True)

# head_dim 64: the size at which the tensor-core prefill attention and the fused decode attention run
D = dict(architectures=["LlamaForCausalLM"], vocab_size=512, hidden_size=128, intermediate_size=320,
         num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, head_dim=64,
         max_position_embeddings=2048, rms_norm_eps=3e-6, rope_theta=250000.0,
         rope_scaling=dict(rope_type="llama3", factor=2.0, low_freq_factor=1.0, high_freq_factor=3.0,
                           original_max_position_embeddings=64),
         tie_word_embeddings=False, eos_token_id=[3])

# head_dim 128 with an odd group of query heads: the size at which the tcgen05 prefill attention runs
E = dict(architectures=["LlamaForCausalLM"], vocab_size=777, hidden_size=192, intermediate_size=448,
         num_hidden_layers=2, num_attention_heads=3, num_key_value_heads=1, head_dim=128,
         max_position_embeddings=2048, rms_norm_eps=1e-5, rope_theta=20000.0, rope_scaling=None,
         tie_word_embeddings=False, eos_token_id=11)

# name -> (config.json contents, weight seed, std of matrices and embeddings)
CONFIGS = {"A": (A, 0, 0.10), "B": (B, 1, 0.08), "C": (C, 2, 0.09), "D": (D, 3, 0.07), "E": (E, 4, 0.06)}
