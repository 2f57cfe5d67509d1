"""LeNet-5: conv5x5 1->6, ReLU, maxpool2; conv5x5 6->16, ReLU, maxpool2; FC 400->120->84->10.
Parity: tests/st/networks/models/lenet.py of the reference (the plumbing / checkpoint round-trip model)."""
from .. import nn


class LeNet5(nn.Cell):
    def __init__(self, num_class=10, num_channel=1):
        super().__init__()
        self.conv1 = nn.Conv2d(num_channel, 6, 5, pad_mode="valid")
        self.conv2 = nn.Conv2d(6, 16, 5, pad_mode="valid")
        self.relu = nn.ReLU()
        self.max_pool2d = nn.MaxPool2d(kernel_size=2, stride=2)
        self.flatten = nn.Flatten()
        self.fc1 = nn.Dense(16 * 5 * 5, 120)
        self.fc2 = nn.Dense(120, 84)
        self.fc3 = nn.Dense(84, num_class)

    def construct(self, x):
        x = self.max_pool2d(self.relu(self.conv1(x)))
        x = self.max_pool2d(self.relu(self.conv2(x)))
        x = self.flatten(x)
        x = self.relu(self.fc1(x))
        x = self.relu(self.fc2(x))
        return self.fc3(x)
