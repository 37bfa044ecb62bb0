"""A complete, minimal training program: logistic regression on two synthetic clusters.

Counterpart of axlearn/experiments/logistic_regression/tutorial.py: a model (a ``Linear`` backbone
and a classification metric), a checkpointable input pipeline, SGD with momentum under a linear
learning-rate decay, an evaler and the trainer configuration, registered as the named config
``LogisticRegression``.

    python -m axlearn_b200.experiments.logistic_regression.tutorial --trainer_dir /tmp/logreg
"""

from __future__ import annotations

import argparse

import numpy as np
import torch

import axlearn_b200 as ax
from axlearn_b200.common import input_pipeline as ip


def _synthesize_data(num_examples: int = 1000, num_features: int = 2, noise_std: float = 0.1, random_seed: int = 42):
    rng = np.random.RandomState(random_seed)
    half = num_examples // 2
    features = np.vstack([rng.normal(loc=[-1.0, -1.0], scale=0.5, size=(half, num_features)),
                          rng.normal(loc=[1.0, 1.0], scale=0.5, size=(half, num_features))])
    features += rng.normal(0, noise_std, features.shape)
    labels = np.hstack([np.zeros(half, dtype=np.int32), np.ones(half, dtype=np.int32)])
    return features.astype(np.float32), labels


def synthetic_source(num_examples: int = 1000, random_seed: int = 42, shuffle_and_repeat: bool = True):
    """``(shard_index, shard_count) -> Stage`` of ``{"features": [2], "label": []}`` examples."""

    def build(shard_index: int, shard_count: int) -> ip.Stage:
        features, labels = _synthesize_data(num_examples=num_examples, random_seed=random_seed)
        examples = [{"features": features[i], "label": labels[i]} for i in range(len(features))]
        return ip.read(ip.ListSource(examples), shuffle=shuffle_and_repeat, seed=random_seed,
                       num_epochs=None if shuffle_and_repeat else 1, shard_index=shard_index, shard_count=shard_count)

    return build


class LogisticRegressionModel(ax.BaseModel):
    @ax.config_class
    class Config(ax.BaseModel.Config):
        backbone: ax.Required[ax.InstantiableConfig] = ax.REQUIRED

    def __init__(self, cfg, *, parent=None):
        super().__init__(cfg, parent=parent)
        self._add_child("backbone", cfg.backbone)
        self._add_child("metric", ax.layers.ClassificationMetric.default_config().set(num_classes=2))

    def predict(self, input_batch: dict) -> dict:
        return {"logits": self.backbone(input_batch["features"])}

    def forward(self, input_batch: dict):
        outputs = self.predict(input_batch)
        logits = outputs["logits"]
        binary_logits = torch.cat([torch.zeros_like(logits), logits], dim=-1)
        loss = self.metric(binary_logits, labels=input_batch["label"].long())
        outputs["binary_logits"] = binary_logits
        outputs["predictions"] = binary_logits.argmax(dim=-1)
        return loss, outputs


def config_input(is_training: bool, global_batch_size: int = 32):
    return ip.PipelineInput.default_config().set(
        source=ax.config_for_function(synthetic_source).set(
            num_examples=1000 if is_training else 200, random_seed=42 if is_training else 123,
            shuffle_and_repeat=is_training),
        global_batch_size=global_batch_size, is_training=is_training, prefetch=2)


def config_logistic_regression_trainer():
    model_cfg = LogisticRegressionModel.default_config().set(
        backbone=ax.layers.Linear.default_config().set(input_dim=2, output_dim=1, bias=True,
                                                       param_partition_spec=(None, None)),
        dtype=torch.float32)
    evaler_cfg = ax.evaler.SpmdEvaler.default_config().set(
        input=config_input(is_training=False), eval_dtype=torch.float32,
        eval_policy=ax.config_for_function(ax.evaler.every_n_steps_policy).set(n=100))
    lr = ax.config_for_function(ax.schedule.polynomial).set(
        begin_value=0.1, end_value=0.01, power=1.0, begin_step=0, end_step=1000)
    optimizer_cfg = ax.config_for_function(ax.optimizers.sgd_optimizer).set(
        learning_rate=lr, momentum=0.9, weight_decay=0.01, decouple_weight_decay=True)
    cfg = ax.SpmdTrainer.default_config().set(
        name="logistic_regression_trainer", mesh_axis_names=("data",), mesh_shape=(1,), model=model_cfg,
        input=config_input(is_training=True), learner=ax.learner.Learner.default_config().set(optimizer=optimizer_cfg),
        evalers={"eval": evaler_cfg}, max_step=1000, train_dtype=None)
    cfg.checkpointer.save_policy = ax.config_for_function(ax.checkpointer.every_n_steps_policy).set(n=200)
    cfg.summary_writer.write_every_n_steps = 10
    return cfg


def named_trainer_configs() -> dict:
    return {"LogisticRegression": config_logistic_regression_trainer}


if __name__ == "__main__":
    parser = argparse.ArgumentParser()
    parser.add_argument("--trainer_dir", required=True)
    parser.add_argument("--max_step", type=int, default=1000)
    args = parser.parse_args()
    trainer = config_logistic_regression_trainer().set(dir=args.trainer_dir, max_step=args.max_step).instantiate(parent=None)
    print(trainer.run(ax.prng.PRNGKey(42)))
