"""CPU oracle (test infrastructure): see ``oracle/muse_layer.py``. Nothing under the product package imports this."""
