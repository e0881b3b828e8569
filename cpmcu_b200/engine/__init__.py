from .step import Chunk, SequenceStep, Stepper, plan_chunks

__all__ = ["Chunk", "SequenceStep", "Stepper", "plan_chunks"]
