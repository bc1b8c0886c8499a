"""The names configs and user code expect from `seqio`, served by this package's data stack."""
from t5x_b200.data.dataset import Dataset, ShardInfo  # noqa: F401
from t5x_b200.data.evaluation import (  # noqa: F401
    Evaluator, JSONLogger, Logger, PyLoggingLogger, TensorBoardLogger)
from t5x_b200.data.feature_converters import (  # noqa: F401
    DecoderFeatureConverter, EncDecFeatureConverter, FeatureConverter, LMFeatureConverter,
    PrefixLMFeatureConverter)
from t5x_b200.data.tasks import (  # noqa: F401
    Feature, Mixture, MixtureRegistry, Task, TaskRegistry, get_dataset, get_mixture_or_task)
from t5x_b200.data.vocabularies import (  # noqa: F401
    ByteVocabulary, PassThroughVocabulary, SentencePieceVocabulary, Vocabulary)

PAD_ID = 0


class loggers:  # namespace parity: seqio.loggers.*
  Logger = Logger
  JSONLogger = JSONLogger
  PyLoggingLogger = PyLoggingLogger
  TensorBoardLogger = TensorBoardLogger
