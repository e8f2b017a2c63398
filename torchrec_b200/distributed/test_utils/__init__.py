"""Test fixtures for sharded models: synthetic inputs, a small sparse + dense model, restricted sharders and a harness that checks
a sharded model against its unsharded twin (``torchrec/distributed/test_utils/``)."""
