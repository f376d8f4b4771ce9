"""The tiny configurations the tests use.  A and B differ in every size and option: layers,
width, heads and groups, head size, feed-forward width (no power of two), vocabulary, rotary
base, the norms' eps, tied or untied output matrix, longest position, page size."""

TINY_A = dict(architectures=["LlamaForCausalLM"], hidden_size=64, num_hidden_layers=2,
              num_attention_heads=4, num_key_value_heads=2, head_dim=16, intermediate_size=176,
              vocab_size=256, rope_theta=10000.0, rms_norm_eps=1e-5, tie_word_embeddings=False,
              max_position_embeddings=128, torch_dtype="float32")
TINY_B = dict(architectures=["LlamaForCausalLM"], hidden_size=256, num_hidden_layers=3,
              num_attention_heads=8, num_key_value_heads=1, head_dim=32, intermediate_size=688,
              vocab_size=512, rope_theta=500000.0, rms_norm_eps=1e-6, tie_word_embeddings=True,
              max_position_embeddings=256, torch_dtype="float32")
# sizes that are no power of two anywhere, a head size that is not hidden/heads, 3 groups
TINY_C = dict(architectures=["LlamaForCausalLM"], hidden_size=120, num_hidden_layers=2,
              num_attention_heads=6, num_key_value_heads=3, head_dim=48, intermediate_size=200,
              vocab_size=331, rope_theta=50000.0, rms_norm_eps=3e-6, tie_word_embeddings=False,
              max_position_embeddings=640, torch_dtype="float32")
# shapes that select the kernels of the full-size models: head size 128 (tcgen05 attention, the
# decode attention that rotates and stores itself), widths that are multiples of 512 (the
# persistent small-batch product), a vocabulary that is no power of two
TINY_D = dict(architectures=["LlamaForCausalLM"], hidden_size=1024, num_hidden_layers=2,
              num_attention_heads=8, num_key_value_heads=2, head_dim=128, intermediate_size=1536,
              vocab_size=1000, rope_theta=500000.0, rms_norm_eps=1e-5, tie_word_embeddings=False,
              max_position_embeddings=2048, torch_dtype="float32")
PAGE_SIZE = {"A": 16, "B": 8, "C": 16, "D": 16}
SEED = {"A": 0, "B": 1, "C": 2, "D": 3}
CONFIGS = {"A": TINY_A, "B": TINY_B, "C": TINY_C, "D": TINY_D}
