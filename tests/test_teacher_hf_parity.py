"""The T5-style teacher against HF `T5EncoderModel` (what the reference wraps,
src/nanoplm/distillation/models/teacher/prott5.py:14-70) with the same random weights, on CPU."""
import pytest
import torch

transformers = pytest.importorskip("transformers")


def test_teacher_loads_hf_t5_encoder_weights_and_reproduces_its_output():
    from transformers import T5Config, T5EncoderModel
    from nanoplm_b200.config.schema import TeacherConfig
    from nanoplm_b200.models.teacher import T5EncoderTeacher
    geom = dict(vocab_size=128, d_model=64, d_kv=16, d_ff=128, num_layers=3, num_heads=4)
    torch.manual_seed(0)
    hf = T5EncoderModel(T5Config(relative_attention_num_buckets=32, relative_attention_max_distance=128,
                                 dropout_rate=0.0, feed_forward_proj="relu", **geom)).float().eval()
    own = T5EncoderTeacher(TeacherConfig(**geom), random_init=True).float().eval()
    theirs = hf.state_dict()
    # HF lists the tied input embedding twice (shared.weight and encoder.embed_tokens.weight)
    assert set(theirs) - set(own.state_dict()) <= {"encoder.embed_tokens.weight"}
    assert set(own.state_dict()) <= set(theirs)
    own.load_state_dict({k: v for k, v in theirs.items() if k in own.state_dict()}, strict=True)
    ids = torch.randint(3, 120, (3, 40))
    mask = torch.ones_like(ids)
    mask[1, 25:] = 0
    mask[2, 7:] = 0
    with torch.no_grad():
        a = hf(input_ids=ids, attention_mask=mask).last_hidden_state
        b = own(ids, mask)
        b = b["last_hidden_state"] if isinstance(b, dict) else getattr(b, "last_hidden_state", b)
    keep = mask.bool()
    assert (a[keep] - b[keep]).abs().max().item() < 2e-5 * max(1.0, a[keep].abs().max().item())
