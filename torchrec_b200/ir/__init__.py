"""Serialisable form of the embedding modules for ``torch.export``: metadata goes into a buffer, the forward becomes one opaque op."""
