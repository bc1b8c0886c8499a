"""In-repo stand-in for the data stack the reference gets from SeqIO / tf.data:
vocabularies, feature converters, a task registry, a checkpointable batch iterator, an
evaluator, and the synthetic span-corruption source used for benchmarks."""
from t5x_b200.data.dataset import Dataset, ShardInfo  # noqa: F401
from t5x_b200.data.feature_converters import (  # noqa: F401
    DecoderFeatureConverter, EncDecFeatureConverter, FeatureConverter, PrefixLMFeatureConverter)
from t5x_b200.data.tasks import (  # noqa: F401
    Feature, MixtureRegistry, Task, TaskRegistry, get_dataset, get_mixture_or_task)
from t5x_b200.data.vocabularies import (  # noqa: F401
    ByteVocabulary, PassThroughVocabulary, SentencePieceVocabulary, Vocabulary)
