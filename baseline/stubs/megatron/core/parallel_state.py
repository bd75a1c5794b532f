"""Parallel state of a pure tensor-parallel training job: the tensor-parallel
group is the default process group, every other parallel size is 1."""

import torch.distributed as dist


def _world():
    return dist.get_world_size() if dist.is_initialized() else 1


def _rank():
    return dist.get_rank() if dist.is_initialized() else 0


def get_tensor_model_parallel_world_size():
    return _world()


def get_tensor_model_parallel_rank():
    return _rank()


def get_tensor_model_parallel_group():
    return dist.group.WORLD


def get_data_parallel_world_size():
    return 1


def get_data_parallel_rank():
    return 0


def get_pipeline_model_parallel_world_size():
    return 1


def get_pipeline_model_parallel_rank():
    return 0


def get_expert_model_parallel_world_size():
    return 1


def get_expert_model_parallel_rank():
    return 0


def get_expert_tensor_parallel_world_size():
    return 1


def get_expert_tensor_parallel_rank():
    return 0


def get_context_parallel_world_size():
    return 1


def get_context_parallel_rank():
    return 0
