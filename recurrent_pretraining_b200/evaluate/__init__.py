"""Evaluation helpers: checkpoint conversion, an lm-eval compatible scorer, depth-comparison chat, step histograms."""
