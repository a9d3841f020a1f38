"""naivert_b200: a Blackwell (sm_100a) single-stream speculative-decoding inference engine."""
__version__ = "0.1.0"
