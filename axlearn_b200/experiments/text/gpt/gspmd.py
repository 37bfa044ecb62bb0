"""The 16B pipelined configuration of the GSPMD paper (arXiv:2105.04663, table 4), for
performance testing of pipeline parallelism.

Parity target in the reference: axlearn/experiments/text/gpt/gspmd.py:37-110 -- 64 layers, width
4096, 64 heads, ReLU feed-forward of 4x width, vocabulary 32K, sequence length 1024, two pipeline
stages x 16 micro-batches (GPipe schedule), Adafactor (momentum 0.9, clipping 5, decay-rate
schedule ``1 - t^-0.8``), global batch 512, mesh ``pipeline=2 x data=-1 x model=8``.  The
reference's "stream" schedule variant is not built.
"""

from __future__ import annotations

from axlearn_b200.common import schedule
from axlearn_b200.common.attention import scaled_hidden_dim
from axlearn_b200.common.config import config_for_function
from axlearn_b200.common.embedding import TransformerTextEmbeddings
from axlearn_b200.common.layers import RMSNorm
from axlearn_b200.common.learner import Learner
from axlearn_b200.common.optimizers import adafactor_optimizer
from axlearn_b200.common.pipeline import PipelinedTransformerLayer
from axlearn_b200.experiments.text.gpt.common import MESH_AXIS_NAMES, get_trainer_config_fn, mesh_shape_from_axes
from axlearn_b200.experiments.text.gpt.common import model_config as common_model_config

_VOCAB_SIZE = 32 * 1024
_MAX_SEQUENCE_LENGTH = 1024
_MAX_STEP = 100_000


def model_config(*, num_layers: int = 64, hidden_dim: int = 128 * 32, num_heads: int = 64, num_stages: int = 2,
                 num_microbatches: int = 16, vocab_size: int = _VOCAB_SIZE):
    stack_cfg = PipelinedTransformerLayer.default_config().set(num_stages=num_stages, num_microbatches=num_microbatches)
    return common_model_config(
        num_layers=num_layers, hidden_dim=hidden_dim, num_heads=num_heads, stack_cfg=stack_cfg, vocab_size=vocab_size,
        ffn_dim=scaled_hidden_dim(4), activation_fn="nn.relu",
        normalization=RMSNorm.default_config().set(forward_dtype=None), emb_cfg=TransformerTextEmbeddings.default_config())


def learner_config() -> Learner.Config:
    return Learner.default_config().set(optimizer=config_for_function(adafactor_optimizer).set(
        learning_rate=config_for_function(schedule.adafactor).set(scale=1e-3), b1=0.9,
        b2=config_for_function(schedule.adafactor_decay_rate), multiply_by_parameter_scale=False,
        clipping_threshold=5, weight_decay=1e-3, weight_decay_scale_by_learning_rate_exponent=1))


def trainer_configs() -> dict:
    def full():
        return get_trainer_config_fn(
            model_cfg=model_config(), learner_cfg=learner_config(), max_step=_MAX_STEP, train_batch_size=512,
            max_sequence_length=_MAX_SEQUENCE_LENGTH, vocab_size=_VOCAB_SIZE,
            mesh_shape=mesh_shape_from_axes(pipeline=2, data=-1, model=8), mesh_axis_names=MESH_AXIS_NAMES)()

    def test():
        return get_trainer_config_fn(
            model_cfg=model_config(num_layers=4, hidden_dim=32, num_heads=4, num_microbatches=2, vocab_size=64),
            learner_cfg=learner_config(), max_step=20, train_batch_size=4, max_sequence_length=16, vocab_size=64,
            mesh_shape=mesh_shape_from_axes(), mesh_axis_names=MESH_AXIS_NAMES)()

    return {"gspmd-16B-2x16x8": full, "gspmd-test": test}
