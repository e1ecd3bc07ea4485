from .decoder import DecoderModel, expected_tensors
