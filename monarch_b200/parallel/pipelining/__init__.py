"""Pipeline parallelism: schedule IR (GPipe, 1F1B, interleaved 1F1B, ZB-H1), a simulator
and the runtime that executes a schedule over tensor-parallel stage engines with NCCL
point-to-point transfers."""
from .runtime import PipelineTrainer, build_mesh_groups  # noqa: F401
from .schedule_ir import (Action, add_communication, bubble_fraction, dump_chrome_trace,  # noqa: F401
                          gpipe, interleaved_1f1b, one_f_one_b, simulate, validate,
                          zero_bubble_h1)
