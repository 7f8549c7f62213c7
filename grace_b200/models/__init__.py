"""Model zoo used by the examples and benchmarks (plain ``torch.nn``)."""
from .resnet_cifar import resnet20, resnet9
from .resnet import resnet50
from .vgg import vgg16
from .bert import bert_large, bert_tiny, BertForPreTraining
from .mnist import MnistNet

__all__ = ["resnet20", "resnet9", "resnet50", "vgg16", "bert_large", "bert_tiny", "BertForPreTraining", "MnistNet"]
