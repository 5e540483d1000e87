// TEST INFRASTRUCTURE. Stand-in for the one external header the reference's test helper includes
// (device/cuda_device.hpp of its un-vendored infrastructure library). It only has to provide
// sci::DeviceManager::Instance().get_device(type, id), which the helper uses for host staging.
#pragma once

#include <memory>

#include "device/device.hpp"

namespace sci {

class DeviceManager {
public:
    static DeviceManager& Instance() {
        static DeviceManager manager;
        return manager;
    }
    std::shared_ptr<Device> get_device(DeviceType, int) {
        return std::shared_ptr<Device>(&StubHostDevice(), [](Device*) {});
    }
};

}  // namespace sci
