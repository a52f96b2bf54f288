"""Speech models: audio input, log-mel features, FastConformer encoders, transducer decoding, transcripts."""
from .audio import LogMel, LogMelConfig, load_audio, read_wav, resample, write_wav  # noqa: F401
from .parakeet import ParakeetModel, ParakeetSpec, TdtDecoder, TdtTrajectory, parakeet_tiny, transcribe  # noqa: F401
from .transcript import TextSegment, Transcription, tdt_cues, word_segments  # noqa: F401
