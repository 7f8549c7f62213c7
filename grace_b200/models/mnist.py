"""Small MNIST CNN of the reference's Horovod example
(``examples/torch/pytorch_mnist.py:76-92``): two 5x5 convs, dropout, two FCs."""
from torch import nn
import torch.nn.functional as F


class MnistNet(nn.Module):
    def __init__(self):
        super().__init__()
        self.conv1 = nn.Conv2d(1, 10, 5)
        self.conv2 = nn.Conv2d(10, 20, 5)
        self.drop = nn.Dropout2d()
        self.fc1 = nn.Linear(320, 50)
        self.fc2 = nn.Linear(50, 10)

    def forward(self, x):
        x = F.relu(F.max_pool2d(self.conv1(x), 2))
        x = F.relu(F.max_pool2d(self.drop(self.conv2(x)), 2))
        x = F.dropout(F.relu(self.fc1(x.view(-1, 320))), training=self.training)
        return F.log_softmax(self.fc2(x), dim=1)
