from .client import RolloutClient, VLLMClient, chunk_list
from .generation import RolloutGeneration, VLLMGeneration, extract_logprobs
