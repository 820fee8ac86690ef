"""Shared fixtures: two tiny configurations of the architecture that differ in every size and
option, their random model folders (made in a temporary folder) and the plain
implementation's view of them."""
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (run with -m gpu on a GPU box)")


def tiny_a():
    from mormot2_ai_b200 import Qwen3Config
    return Qwen3Config(vocab_size=256, hidden_size=64, num_hidden_layers=2,
                       num_attention_heads=4, num_key_value_heads=2, head_dim=16,
                       intermediate_size=128, max_position_embeddings=128, rms_norm_eps=1e-6,
                       rope_theta=10000.0, tie_word_embeddings=True)


def tiny_b():
    """Differs from tiny A in every size and option: 3 layers, MQA (6 heads on 1 KV head),
    head_dim 32 with q width 192 != hidden 96, sizes that are no power of two (96, 320, 509),
    other eps and theta, untied head, and a sliding window of 24 in the middle layer."""
    from mormot2_ai_b200 import Qwen3Config
    return Qwen3Config(vocab_size=509, hidden_size=96, num_hidden_layers=3,
                       num_attention_heads=6, num_key_value_heads=1, head_dim=32,
                       intermediate_size=320, max_position_embeddings=256, rms_norm_eps=1e-5,
                       rope_theta=1e6, tie_word_embeddings=False, layer_windows=(0, 24, 0))


def tiny_c():
    """Heads of 64 values (the smallest size the tensor-core attention kernels take), groups of
    two, q width 256 != hidden 128, a window of 70 in the first layer, tied head."""
    from mormot2_ai_b200 import Qwen3Config
    return Qwen3Config(vocab_size=384, hidden_size=128, num_hidden_layers=2,
                       num_attention_heads=4, num_key_value_heads=2, head_dim=64,
                       intermediate_size=192, max_position_embeddings=320, rms_norm_eps=1e-6,
                       rope_theta=5e5, tie_word_embeddings=True, layer_windows=(70, 0))


def tiny_d():
    """Heads of 128 values (the size of the tcgen05 attention kernel), three query heads on one
    KV head, a hidden size below the q width, a window of 100 in the second layer."""
    from mormot2_ai_b200 import Qwen3Config
    return Qwen3Config(vocab_size=320, hidden_size=192, num_hidden_layers=2,
                       num_attention_heads=3, num_key_value_heads=1, head_dim=128,
                       intermediate_size=256, max_position_embeddings=384, rms_norm_eps=1e-6,
                       rope_theta=1e4, tie_word_embeddings=False, layer_windows=(0, 100))


TINY = {"A": (tiny_a, 0, 0.02, [5, 11, 17], 8), "B": (tiny_b, 1, 0.03, [1, 7, 30, 64], 12),
        "C": (tiny_c, 2, 0.04, [3, 66, 129], 6), "D": (tiny_d, 3, 0.04, [2, 130, 200], 5)}


class TinyModel:
    def __init__(self, name, folder):
        from mormot2_ai_b200 import write_random_model
        from tests.plain import qwen3_plain as plain
        make, seed, std, lens, decode = TINY[name]
        self.name, self.config, self.seed = name, make(), seed
        self.prompt_lens, self.decode_steps = lens, decode
        self.folder = write_random_model(folder, self.config, seed, std=std, norm_std=0.1)
        self.plain_config, self.plain_weights = plain.read_model_folder(self.folder)
        self.plain = plain

    def tokens(self, n, seed=0):
        rng = np.random.default_rng(1000 * self.seed + seed)
        return rng.integers(0, self.config.vocab_size, n).tolist()

    def reference(self, ids):
        return self.plain.forward(self.plain_config, self.plain_weights, ids)


@pytest.fixture(scope="session", params=["A", "B", "C", "D"])
def tiny(request, tmp_path_factory):
    return TinyModel(request.param, str(tmp_path_factory.mktemp("tiny_" + request.param)))


@pytest.fixture(scope="session")
def tiny_a_model(tmp_path_factory):
    return TinyModel("A", str(tmp_path_factory.mktemp("tiny_A_only")))


@pytest.fixture(scope="session")
def tiny_b_model(tmp_path_factory):
    return TinyModel("B", str(tmp_path_factory.mktemp("tiny_B_only")))


# Tolerances, fixed once and never widened to pass: the largest difference of a logit from the
# plain implementation's. float32: relative to the largest logit of the comparison (at least
# 1); both sides round to float32 at the same places and differ by summation order only.
# bfloat16: relative to the standard deviation of the plain logits of the comparison: every
# activation between kernels is rounded to 8 bits of mantissa, which moves a logit by a small
# share of the spread of the logits, whatever their size; a wrong or missing key, token or
# page moves it by a large share. MORMOT_TOL_RECORD names a file that every comparison is
# appended to (how far inside the bound the engine runs).
TOL = {"float32": 1e-5, "bfloat16": 6e-2}


def close(got, want, dtype):
    got, want = np.asarray(got, dtype=np.float64), np.asarray(want, dtype=np.float64)
    assert got.shape == want.shape, (got.shape, want.shape)
    if dtype == "bfloat16":
        scale = float(want.std())
    else:
        scale = max(1.0, float(np.abs(want).max()))
    err = float(np.abs(got - want).max())
    record = os.environ.get("MORMOT_TOL_RECORD")
    if record:
        test = os.environ.get("PYTEST_CURRENT_TEST", "").split(" ")[0]
        with open(record, "a") as f:
            f.write(f"{dtype}\t{err / scale:.3e}\t{err:.3e}\t{scale:.3e}\t{test}\n")
    return err <= TOL[dtype] * scale, err / scale
