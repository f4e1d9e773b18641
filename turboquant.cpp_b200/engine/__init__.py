"""The engine: loading, the step function, the generation loop."""
from .step import Engine, StepEntry, StepError
from .loading import build_model, load_model, random_model, write_random_folder
