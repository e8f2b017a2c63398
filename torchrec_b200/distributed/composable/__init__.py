"""Composable-API pieces of the sharded embedding modules (``torchrec/distributed/composable/``)."""
