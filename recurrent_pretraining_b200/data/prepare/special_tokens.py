"""The tokenizer's special-token inventory.  The training and inference code depends on four of them by id
(vocab 65536: ``<|begin_text|>`` 65504, ``<|end_text|>`` 65505, ``<|end_turn|>`` 65508, ``<|pad|>`` 65509,
recpre/raven_modeling_minimal.py:1929-1942), so the specials occupy the LAST ids of the vocabulary, in this order
(scripts/tokenizer_generation.py:494-540)."""

SPECIAL_TOKENS = [
    "<|begin_text|>", "<|end_text|>", "<|begin_header|>", "<|end_header|>", "<|end_turn|>", "<|pad|>",
    "<|fim_prefix|>", "<|fim_middle|>", "<|fim_suffix|>", "<|fim_pad|>", "<|...|>", "<|del|>",
    *[f"<|c_{i}|>" for i in range(10)],
]
assert len(SPECIAL_TOKENS) == 22
# the remaining ids up to 32 are reserved markers for tools / control
SPECIAL_TOKENS += ["<|?|>", "<|&|>", "<|!|>", "<|-|>", "<|+|>", "<|interrupt|>", "<|tool_out|>", "<|end_tool|>",
                   "<|tool_in|>", "<|end_tool_in|>"]
N_SPECIAL = 32


def special_token_ids(vocab_size: int = 65536) -> dict:
    base = vocab_size - N_SPECIAL
    return {tok: base + i for i, tok in enumerate(SPECIAL_TOKENS)}
