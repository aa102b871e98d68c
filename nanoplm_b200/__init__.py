"""nanoplm_b200: Blackwell-native protein language model pretraining and distillation."""
import os as _os

# Every kernel of this package takes its sizes at run time and the models cut padding off their
# batches, so tensor sizes change from micro-batch to micro-batch. Expandable segments keep the
# caching allocator from fragmenting (and from calling cudaMalloc in the steady state) under such
# a load; the setting has to be in place before the first CUDA allocation of the process.
# The reference sets the same variable in its training pipeline (pure_pipeline.py, start of
# run_pure_pretraining). An explicit user setting wins.
_os.environ.setdefault("PYTORCH_ALLOC_CONF", "expandable_segments:True")

__version__ = "0.1.0"
