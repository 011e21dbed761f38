from . import transformers
