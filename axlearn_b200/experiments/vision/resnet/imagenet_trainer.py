"""ResNet on ImageNet: the named trainer configs ``ResNet-{Test,Testb,18,34,50,50-ema,101,152}``.

Counterpart of axlearn/experiments/vision/resnet/{common.py, imagenet_trainer.py} and
axlearn/experiments/vision/imagenet/common.py: 90 epochs of SGD with momentum 0.9, L2 weight decay
1e-4 on everything but the norms, cosine decay with 5 warm-up epochs and a peak learning rate of
``0.1 * batch / 256``; Kaiming-normal (fan-out) weights; evaluation and a checkpoint every 10 epochs.
Without a dataset directory the inputs are random images.
"""

from __future__ import annotations

import math
from typing import Callable, Optional

import torch

from axlearn_b200.common import checkpointer, evaler, learner, optimizers, param_init, schedule
from axlearn_b200.common.config import config_for_function
from axlearn_b200.common.evaler import SpmdEvaler
from axlearn_b200.common.input_fake import FakeImageInput
from axlearn_b200.common.trainer import SpmdTrainer
from axlearn_b200.vision import image_classification
from axlearn_b200.vision.resnet import ResNet, named_resnet_config

NUM_TRAIN_EXAMPLES = 1_281_167
NUM_CLASSES = 1_000


def input_config(*, split: str, global_batch_size: int, total_num_batches: Optional[int] = None):
    """Random images stand in for the dataset; ``split`` only seeds them differently."""
    return FakeImageInput.default_config().set(
        global_batch_size=global_batch_size, is_training=split.startswith("train") and "[" not in split,
        num_classes=NUM_CLASSES, seed=sum(map(ord, split)), total_num_batches=total_num_batches)


def learner_config(*, learning_rate, ema_decay: Optional[float] = None):
    per_param_decay = config_for_function(optimizers.per_param_scale_by_path).set(
        description="weight_decay_scale", scale_by_path=[(".*norm.*", 0)])
    optimizer = config_for_function(optimizers.sgd_optimizer).set(
        learning_rate=learning_rate, decouple_weight_decay=False, momentum=0.9, weight_decay=1e-4,
        weight_decay_per_param_scale=per_param_decay)
    cfg = learner.Learner.default_config().set(optimizer=optimizer)
    if ema_decay:
        cfg.ema.decay = ema_decay
    return cfg


def model_config():
    cfg = image_classification.ImageClassificationModel.default_config().set(dtype=torch.float32)
    cfg.param_init = param_init.DefaultInitializer.default_config().set(init_by_param_name={
        param_init.PARAM_REGEXP_WEIGHT: param_init.WeightInitializer.default_config().set(
            fan="fan_out", distribution="normal", scale=math.sqrt(2))})
    return cfg


def _get_config_fn(backbone, *, train_batch_size: int, ema_decay: Optional[float] = None,
                   compute_dtype: torch.dtype = torch.bfloat16) -> Callable[[], SpmdTrainer.Config]:
    def config_fn():
        steps_per_epoch = NUM_TRAIN_EXAMPLES // train_batch_size
        max_step = steps_per_epoch * 90
        every = steps_per_epoch * 10
        cfg = SpmdTrainer.default_config().set(name="resnet_imagenet", train_dtype=compute_dtype, max_step=max_step)
        cfg.model = model_config().set(backbone=backbone.clone(), num_classes=NUM_CLASSES)
        cfg.input = input_config(split="train", global_batch_size=train_batch_size)
        cfg.evalers = {}
        for name, split in (("eval_train", "train[:50000]"), ("eval_validation", "validation")):
            cfg.evalers[name] = SpmdEvaler.default_config().set(
                input=input_config(split=split, global_batch_size=80, total_num_batches=2),
                eval_policy=config_for_function(evaler.every_n_steps_policy).set(n=every), eval_dtype=compute_dtype)
        cfg.learner = learner_config(
            learning_rate=config_for_function(schedule.cosine_with_linear_warmup).set(
                peak_lr=0.1 * train_batch_size / 256, max_step=max_step, warmup_steps=steps_per_epoch * 5),
            ema_decay=ema_decay)
        cfg.checkpointer.save_policy = config_for_function(checkpointer.every_n_steps_policy).set(n=every)
        cfg.checkpointer.keep_every_n_steps = every
        cfg.summary_writer.write_every_n_steps = 100
        return cfg

    return config_fn


def named_trainer_configs() -> dict:
    r18 = named_resnet_config("resnet18")
    return {
        "ResNet-Test": _get_config_fn(r18.clone(hidden_dim=4, num_blocks_per_stage=[]), train_batch_size=2),
        "ResNet-Testb": _get_config_fn(r18.clone(hidden_dim=4, num_blocks_per_stage=[1]), train_batch_size=256),
        "ResNet-18": _get_config_fn(r18, train_batch_size=1024),
        "ResNet-34": _get_config_fn(named_resnet_config("resnet34"), train_batch_size=1024),
        "ResNet-50": _get_config_fn(named_resnet_config("resnet50"), train_batch_size=1024),
        "ResNet-50-ema": _get_config_fn(named_resnet_config("resnet50"), train_batch_size=1024, ema_decay=0.9999),
        "ResNet-101": _get_config_fn(named_resnet_config("resnet101"), train_batch_size=1024),
        "ResNet-152": _get_config_fn(named_resnet_config("resnet152"), train_batch_size=1024),
    }
