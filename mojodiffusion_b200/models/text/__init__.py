"""Text side: tokenizers (CLIP BPE, byte-level BPE for the Qwen family, SentencePiece unigram for T5) and encoders
(CLIP text transformer, T5 encoder, Qwen3 decoder stack used as an encoder) with the checkpoint key names of the
Hugging Face releases (serenitymojo/tokenizer/*.mojo, serenitymojo/models/text_encoder/{clip,t5,qwen3}_encoder.mojo)."""
from .clip import CLIPTextConfig, CLIPTextEncoder
from .gpt_oss import GptOssConfig, GptOssEncoder
from .qwen3 import Qwen3Config, Qwen3Encoder
from .t5 import T5Config, T5Encoder
from .tokenizers import ByteLevelBPE, CLIPTokenizer, T5Tokenizer
