"""Offline data preparation: tokenizer training, tokenise -> shuffle -> pack -> shard, reshuffle rounds, token counts."""
