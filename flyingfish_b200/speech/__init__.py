"""Speech models: audio input, log-mel features, FastConformer encoders, transducer decoding, transcripts."""
from .audio import LogMel, LogMelConfig, StreamingLogMel, load_audio, read_wav, resample, write_wav  # noqa: F401
from .parakeet import (ParakeetCtcModel, ParakeetCtcSpec, ParakeetModel, ParakeetSpec, TdtDecoder, TdtTrajectory,  # noqa: F401
                       load_model, parakeet_tiny, transcribe, StreamingRecognizer, nemotron_tiny, streaming_tiny)
from .transcript import TextSegment, Transcription, speaker_segments, tdt_cues, to_rttm, word_segments  # noqa: F401
from .canary import CanaryModel, CanarySpec, canary_prompt, canary_tiny  # noqa: F401
from .diarization import DiarizationModel, DiarizationSpec, DiarizationStream, diarization_tiny, select_cache_rows  # noqa: F401
from .multitalker import MultitalkerModel, MultitalkerSpec, MultitalkerStream, transcribe_multitalker  # noqa: F401
