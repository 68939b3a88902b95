"""LeNet-style CNN of the MNIST examples: conv 1->20 5x5, maxpool, conv 20->50 5x5,
maxpool, fc 800->500, ReLU, fc 500->10 (reference: examples/dp/mnist/pytorch/main.py)."""
import torch.nn as nn
import torch.nn.functional as F


class LeNet(nn.Module):
    def __init__(self, classes: int = 10):
        super().__init__()
        self.conv1 = nn.Conv2d(1, 20, 5, 1)
        self.conv2 = nn.Conv2d(20, 50, 5, 1)
        self.fc1 = nn.Linear(4 * 4 * 50, 500)
        self.fc2 = nn.Linear(500, classes)

    def forward(self, x):
        x = F.max_pool2d(F.relu(self.conv1(x)), 2, 2)
        x = F.max_pool2d(F.relu(self.conv2(x)), 2, 2)
        x = F.relu(self.fc1(x.flatten(1)))
        return self.fc2(x)

    def parts(self):
        """Two pipeline / ZeRO units: the convolutional trunk and the classifier."""
        trunk = nn.Sequential(self.conv1, nn.ReLU(), nn.MaxPool2d(2, 2), self.conv2, nn.ReLU(),
                              nn.MaxPool2d(2, 2), nn.Flatten(1))
        head = nn.Sequential(self.fc1, nn.ReLU(), self.fc2)
        return [trunk, head]
