"""Turning logits into the next token."""
