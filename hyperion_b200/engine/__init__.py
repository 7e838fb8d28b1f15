from .batch import BadStep, StepContext, StepEntry

__all__ = ["BadStep", "StepContext", "StepEntry", "ModelRunner"]


def __getattr__(name):
    # the runner imports the model, which imports this package's batch module: resolve it late
    if name == "ModelRunner":
        from .runner import ModelRunner

        return ModelRunner
    raise AttributeError(name)
