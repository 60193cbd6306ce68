"""Entry points of the framework: miner, validator, evaluator, burn (``python neurons/<name>.py``)."""
